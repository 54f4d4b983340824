// Attention of prompt steps over the paged cache on the 5th-generation tensor cores (sm_100a),
// bfloat16, head size 128: S = Q K^T and O += P V as tcgen05.mma with the accumulators in tensor
// memory, K and V pages brought by TMA, softmax in 32-bit by threads that each own one query row.
//
// One block works on one (128 query rows of a sequence, query head).  Keys go by in blocks of 128
// (two cache pages).  Roles:
//   warps 0-7  softmax: threads r and r + 128 own query row r = lane r of tensor memory, 64 columns
//              each.  A thread reads its half row of S (tcgen05.ld), masks, takes the maximum (the two
//              halves meet through shared memory), writes P = 2^(s*c - m*c) as packed bfloat16 back
//              into tensor memory over the scores it has read (tcgen05.st), rescales its half row of O
//              when the reference point m moved, and at the end writes O / l.  m moves lazily (only
//              when the maximum grew by more than 2^8), which spares most rescalings.  At the start
//              the same threads copy the Q tile from shared memory into tensor memory
// Both products take their A operand (Q, P) from tensor memory, so an MMA reads only its B operand
// (K, V) from shared memory: with A in shared memory as well, a 128 x 128 x 16 MMA needs all of the
// 128 bytes a clock that shared memory delivers, and the first version ran at half the rate.
//   warp 8     one lane issues the MMAs: S(j+1) = Q K(j+1)^T is issued BEFORE it waits for P(j), so
//              the tensor cores work on the next scores while the softmax warps are busy (S is
//              double-buffered in tensor memory); then O += P(j) V(j)
//   warp 9     one lane issues the TMA loads: Q once, then K and V of every block into a ring of three
//              stages
// V is read as an MN-major operand (rows of the cache are keys, the MMA contracts over keys), so the
// cache layout [page, kv head, 64 tokens, head size] serves both products as it is.
//
// Masking: key j is visible to the query at position p iff j <= p and (window == 0 or j > p - window).
// Rows of V at or beyond the sequence's length are zeroed in shared memory before P V (their P is
// zero, but 0 * NaN is NaN), scores against such keys are replaced before they are used.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word
// (sx_attn_tc_status) and the block still frees its tensor memory.
//
// The reference's prompt attention is an mma.sync FA-2 kernel for contiguous caches
// (crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_splitq.cu:187-600); it has no tcgen05 path.
#include <cuda.h>
#include "common.cuh"

#define FT_HD 128
#define FT_BM 128                       // query rows of a block
#define FT_BN 128                       // keys of a block
#define FT_SOFTMAX_THREADS 256
#define FT_MMA_WARP 8
#define FT_TMA_WARP 9
#define FT_THREADS 320
#define FT_HALF 64                     // columns of S (and of O) a softmax thread owns
#define FT_CHUNK (128 * 128)            // bytes of [128 rows][64 values]: one swizzled half of a 128 x 128 bf16 tile
#define FT_TILE (2 * FT_CHUNK)          // 32 KB
#define FT_STAGE (2 * FT_TILE)          // K then V
#define FT_KV_STAGES 3                  // K/V blocks in flight: with two, every block waited for its loads (measured 1.85 us a block)
#define FT_SMEM_TILES (FT_KV_STAGES * FT_STAGE)      // Q lands in the last stage's K tile and moves on to tensor memory before that stage is first used
#define FT_SPIN_LIMIT (1u << 26)
#define FT_TMEM_COLS 512
#define FT_COL_S0 0
#define FT_COL_S1 128
#define FT_COL_O 256
#define FT_COL_Q 384                    // Q as packed bf16: 64 columns; P(j) lies over the first 64 columns of S(j)
#define FT_LAZY 8.0f

__device__ __forceinline__ uint32_t ft_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ft_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ft_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ft_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ft_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < FT_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void ft_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void ft_tma_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// shared-memory matrix descriptors, 128-byte swizzle.  K-major (Q, K, P): rows of 128 bytes, groups of
// 8 rows 1024 bytes apart.  MN-major (V): a row of 128 bytes holds 64 values of the N side for one
// key; groups of 8 keys are 1024 bytes apart (stride offset), the next 64 values of N are one
// 16 KB chunk further (leading offset).
__device__ __forceinline__ uint64_t ft_desc_kmajor(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint64_t ft_desc_mnmajor(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)(FT_CHUNK >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D f32, A and B bf16, M x N of the instruction; b_mn: B is MN-major
__host__ __device__ constexpr uint32_t ft_idesc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void ft_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (128 lanes x 8 columns of packed bf16 pairs per K = 16)
__device__ __forceinline__ void ft_mma_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ft_st32u(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// one lane of the (converged) warp
__device__ __forceinline__ bool ft_elect_one() {
  uint32_t is_leader;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(is_leader));
  return is_leader != 0;
}
__device__ __forceinline__ void ft_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ft_ld32(uint32_t taddr, float* r) {
  uint32_t v[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(v[i]);
}
__device__ __forceinline__ void ft_st32(uint32_t taddr, const float* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
        "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
        "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
        "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15])),
        "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])), "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])),
        "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
        "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])), "r"(__float_as_uint(r[27])),
        "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])), "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
      : "memory");
}
// 2^x on the special-function unit: one instruction, -inf -> 0
__device__ __forceinline__ float ft_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t ft_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

enum { FT_B_QFULL = 0, FT_B_KVFULL = 1, FT_B_KVEMPTY = 1 + FT_KV_STAGES, FT_B_SFULL = 1 + 2 * FT_KV_STAGES, FT_B_QREADY = FT_B_SFULL + 2,
       FT_B_PREADY = FT_B_QREADY + 1, FT_B_PVDONE = FT_B_PREADY + 1, FT_B_XCH = FT_B_PVDONE + 1, FT_NBARS = FT_B_XCH + 12 };

__global__ void __launch_bounds__(FT_THREADS, 1) attn_tc_prefill_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ tile_seq,
    const int* __restrict__ tile_q0, const int* __restrict__ cu_seqlens, const int* __restrict__ seq_past,
    const int* __restrict__ seq_lens, const int* __restrict__ block_table, int maxp, int nh, int nkv,
    float scale_log2, int window, int* __restrict__ status) {
  extern __shared__ unsigned char ft_smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ft_smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* kv_s = tiles;                                   // [FT_KV_STAGES][K tile, V tile]
  unsigned char* q_s = kv_s + (FT_KV_STAGES - 1) * FT_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + FT_SMEM_TILES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FT_NBARS);
  float* xch = reinterpret_cast<float*>(tmem_slot + 4);          // [6][128]: the halves' maxima (two buffers), their sums
  const uint32_t bar0 = ft_smem(bars);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Tiles late in a sequence see more keys: they are started first, for all heads (blocks are handed out
  // with x running fastest), so that the short ones fill the tail
  const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
  const int seq = tile_seq[tile], q0 = tile_q0[tile];
  const int kvh = h / (nh / nkv);
  const int t_begin = cu_seqlens[seq], n_new = cu_seqlens[seq + 1] - t_begin;
  const int past = seq_past[seq], len = seq_lens[seq];
  const int rows = min(FT_BM, n_new - q0);
  const int first_pos = past + q0, last_pos = past + q0 + rows - 1;
  const int lo_key = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int kb0 = (lo_key / FT_BN) * FT_BN;
  const int nb = (last_pos + 1 - kb0 + FT_BN - 1) / FT_BN;       // >= 1
  const int* bt = block_table + (size_t)seq * maxp;

  if (threadIdx.x == 0) {
    ft_mbar_init(bar(FT_B_QFULL), 1);
    for (int s = 0; s < FT_KV_STAGES; ++s) {
      ft_mbar_init(bar(FT_B_KVFULL + s), 1);
      ft_mbar_init(bar(FT_B_KVEMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) ft_mbar_init(bar(FT_B_SFULL + s), 1);
    // one arrival per softmax warp (its lane 0, after the warp has synchronised): 256 arrivals on one
    // barrier word cost more than the softmax itself
    ft_mbar_init(bar(FT_B_QREADY), FT_SOFTMAX_THREADS / 32);
    ft_mbar_init(bar(FT_B_PREADY), FT_SOFTMAX_THREADS / 32);
    ft_mbar_init(bar(FT_B_PVDONE), 1);
    for (int s = 0; s < 12; ++s) ft_mbar_init(bar(FT_B_XCH + s), 2);      // the exchanges between warps w and w + 4: [3][4]
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == FT_MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(ft_smem(tmem_slot)), "r"((uint32_t)FT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_trigger();

  if (warp == FT_TMA_WARP) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      ft_mbar_expect_tx(bar(FT_B_QFULL), FT_TILE);
      ft_tma_2d(ft_smem(q_s), &map_q, h * FT_HD, t_begin + q0, bar(FT_B_QFULL));
      ft_tma_2d(ft_smem(q_s + FT_CHUNK), &map_q, h * FT_HD + 64, t_begin + q0, bar(FT_B_QFULL));
      for (int j = 0; j < nb; ++j) {
        const int s = j % FT_KV_STAGES, u = j / FT_KV_STAGES;
        if (!ft_mbar_wait(bar(FT_B_KVEMPTY + s), (u & 1) ^ 1)) { sx_set_status(status, 1); break; }
        if (j == FT_KV_STAGES - 1 && !ft_mbar_wait(bar(FT_B_QREADY), 0)) { sx_set_status(status, 1); break; }      // Q has left this stage
        ft_mbar_expect_tx(bar(FT_B_KVFULL + s), FT_STAGE);
        const uint32_t k_dst = ft_smem(kv_s + s * FT_STAGE), v_dst = k_dst + FT_TILE;
        const int key0 = kb0 + j * FT_BN;
#pragma unroll
        for (int hp = 0; hp < 2; ++hp) {
          const int pi = (key0 >> 6) + hp;
          // a page beyond the sequence's keys is never looked up: page 0 stands in, its keys are masked
          const int page = (pi * 64 < len && pi < maxp) ? bt[pi] : 0;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            ft_tma_4d(k_dst + c * FT_CHUNK + hp * 8192, &map_k, c * 64, 0, kvh, page, bar(FT_B_KVFULL + s));
            ft_tma_4d(v_dst + c * FT_CHUNK + hp * 8192, &map_v, c * 64, 0, kvh, page, bar(FT_B_KVFULL + s));
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == FT_MMA_WARP) {
    // ------------------------------ MMA issuer ------------------------------
    // The WHOLE warp walks the key blocks, so that addresses and descriptors are computed in uniform control
    // flow and stay in uniform registers, and one elected lane issues.  (With one lane branching off alone every
    // tcgen05.mma cost tens of nanoseconds to issue, more than the instruction takes to run.)
    constexpr uint32_t idesc_qk = ft_idesc(FT_BM, FT_BN, false);
    constexpr uint32_t idesc_pv = ft_idesc(FT_BM, FT_HD, true);
    const bool leader = ft_elect_one();
    const uint32_t kv_addr = ft_smem(kv_s);
    // Q is in tensor memory once the softmax threads have copied it there
    bool ok = __all_sync(0xffffffffu, ft_mbar_wait(bar(FT_B_QREADY), 0));
    if (!ok && leader) sx_set_status(status, 2);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    // MMAs run in the order they are issued, so S(j+2) = Q K(j+2)^T, issued after P(j) V(j), does not
    // overwrite P(j), which lies over S(j)
    auto issue_qk = [&](int j) -> bool {
      const int ks = j % FT_KV_STAGES, ku = j / FT_KV_STAGES, s = j & 1;
      if (!__all_sync(0xffffffffu, ft_mbar_wait(bar(FT_B_KVFULL + ks), ku & 1))) {
        if (leader) sx_set_status(status, 3);
        return false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint64_t dk = ft_desc_kmajor(kv_addr + ks * FT_STAGE);
      const uint32_t d = tmem_base + (s ? FT_COL_S1 : FT_COL_S0), qa = tmem_base + FT_COL_Q;
      if (leader) {
#pragma unroll
        for (int k = 0; k < FT_HD / 16; ++k)       // the descriptor's address counts 16-byte units
          ft_mma_ta(d, qa + k * 8, dk + (((k >> 2) * FT_CHUNK + (k & 3) * 32) >> 4), idesc_qk, k != 0);
        ft_commit(bar(FT_B_SFULL + s));
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < nb && ok; ++j) {
      if (j + 1 < nb) ok = issue_qk(j + 1);
      if (!ok) break;
      ok = __all_sync(0xffffffffu, ft_mbar_wait(bar(FT_B_PREADY), j & 1));
      if (!ok) {
        if (leader) sx_set_status(status, 5);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int ks = j % FT_KV_STAGES;
      const uint32_t pa = tmem_base + ((j & 1) ? FT_COL_S1 : FT_COL_S0), o_acc = tmem_base + FT_COL_O;
      const uint64_t dv = ft_desc_mnmajor(kv_addr + ks * FT_STAGE + FT_TILE);
      const uint32_t acc = j != 0;
      if (leader) {
#pragma unroll
        for (int k = 0; k < FT_BN / 16; ++k)       // P: 8 columns (16 keys) further; V: 16 rows of 128 bytes further
          ft_mma_ta(o_acc, pa + k * 8, dv + k * (2048 >> 4), idesc_pv, acc | (k != 0));
        ft_commit(bar(FT_B_PVDONE));
        ft_commit(bar(FT_B_KVEMPTY + ks));
      }
      __syncwarp();
    }
    __syncwarp();
  } else {
    // ---------------- softmax: threads r and r + 128 own query row r, 64 columns each ----------------
    const int r = threadIdx.x & 127, hf = threadIdx.x >> 7;      // row; which half of the columns
    const uint32_t t_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const int pos = r < rows ? past + q0 + r : -1;
    float m = -INFINITY, l = 0.f;                                 // l: this thread's columns only
    bool ok = true;
    // this thread's half row of Q (64 values = one swizzled chunk row) from shared into tensor memory
    if (!ft_mbar_wait(bar(FT_B_QFULL), 0)) { sx_set_status(status, 6); ok = false; }
    {
      uint32_t qv[32];
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const uint4 v = *reinterpret_cast<const uint4*>(q_s + hf * FT_CHUNK + r * 128 + ((p ^ (r & 7)) << 4));
        qv[p * 4] = v.x; qv[p * 4 + 1] = v.y; qv[p * 4 + 2] = v.z; qv[p * 4 + 3] = v.w;
      }
      ft_st32u(t_row + FT_COL_Q + hf * 32, qv);
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) ft_mbar_arrive(bar(FT_B_QREADY));
    }
    for (int j = 0; j < nb && ok; ++j) {
      const int s = j & 1, u = j >> 1;
      if (!ft_mbar_wait(bar(FT_B_SFULL + s), u & 1)) { sx_set_status(status, 6); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      float sc[FT_HALF];
#pragma unroll
      for (int c = 0; c < FT_HALF / 32; ++c) ft_ld32(t_row + (s ? FT_COL_S1 : FT_COL_S0) + hf * FT_HALF + c * 32, sc + c * 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");

      const int key0 = kb0 + j * FT_BN;
      const bool need_mask = key0 + FT_BN - 1 > first_pos || (window > 0 && key0 <= last_pos - window);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < FT_HALF; ++i) {
          const int ja = key0 + hf * FT_HALF + i;
          const bool vis = ja <= pos && (window == 0 || ja > pos - window);
          sc[i] = vis ? sc[i] : -INFINITY;
        }
      }
      // the maximum of this thread's columns with 8 independent chains, then of the row through shared memory
      float mxs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mxs[i] = sc[i];
#pragma unroll
      for (int i = 8; i < FT_HALF; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], sc[i]);
      const float hmax = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      xch[(s * 2 + hf) * FT_BM + r] = hmax;
      __syncwarp();                                // (a bounded wait instead of a named barrier: a warp that gave up does not hang its partner)
      if (lane == 0) ft_mbar_arrive(bar(FT_B_XCH + s * 4 + (warp & 3)));
      if (!ft_mbar_wait(bar(FT_B_XCH + s * 4 + (warp & 3)), u & 1)) { sx_set_status(status, 9); ok = false; break; }
      const float bmax = fmaxf(hmax, xch[(s * 2 + (hf ^ 1)) * FT_BM + r]);
      // The reference point m moves only when the maximum has grown by more than FT_LAZY (in the exponent's
      // units): until then p = 2^(s*c - m*c) may exceed 1 by at most 2^FT_LAZY, which float32 sums and
      // bfloat16 P hold without loss, and O needs no rescaling.  The final O / l is the same either way.
      // Both threads of a row see the same bmax and m, so they decide alike.
      float corr = 1.f;
      if (bmax != -INFINITY && (m == -INFINITY || (bmax - m) * scale_log2 > FT_LAZY)) {
        corr = (m == -INFINITY) ? 0.f : ft_ex2((m - bmax) * scale_log2);
        m = bmax;
      }
      const float ms = (m == -INFINITY) ? 0.f : m * scale_log2;
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[FT_HALF / 2];
#pragma unroll
      for (int i = 0; i < FT_HALF; i += 2) {
        const float p0 = ft_ex2(fmaf(sc[i], scale_log2, -ms));
        const float p1 = ft_ex2(fmaf(sc[i + 1], scale_log2, -ms));
        sums[(i >> 1) & 3] += p0 + p1;
        pk[i >> 1] = ft_pack(p0, p1);
      }
      l = l * corr + ((sums[0] + sums[1]) + (sums[2] + sums[3]));

      // P goes over the scores of this block (every thread of the row has read its scores: the
      // exchange of the maxima came after the loads); O is free once the previous block's P V is done
      ft_st32u(t_row + (s ? FT_COL_S1 : FT_COL_S0) + hf * 32, pk);
      if (j > 0 && !ft_mbar_wait(bar(FT_B_PVDONE), (j - 1) & 1)) { sx_set_status(status, 7); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      // rows of V at or beyond the sequence's length (thread r stands for key r of the block here,
      // and hf for the half of the head's values)
      if (key0 + r >= len) {
        unsigned char* vrow = kv_s + (j % FT_KV_STAGES) * FT_STAGE + FT_TILE + hf * FT_CHUNK + r * 128;
#pragma unroll
        for (int p = 0; p < 8; ++p) *reinterpret_cast<uint4*>(vrow + p * 16) = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // the zeroed rows, for the tensor cores
      }
      // O *= corr (this thread's 64 columns), when some row of this warp moved its reference point
      if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < FT_HALF / 32; ++c) {
          float o[32];
          ft_ld32(t_row + FT_COL_O + hf * FT_HALF + c * 32, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= corr;
          ft_st32(t_row + FT_COL_O + hf * FT_HALF + c * 32, o);
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) ft_mbar_arrive(bar(FT_B_PREADY));
    }
    // the row's sum: both halves
    xch[(4 + hf) * FT_BM + r] = l;
    __syncwarp();
    if (lane == 0) ft_mbar_arrive(bar(FT_B_XCH + 8 + (warp & 3)));
    if (ok && !ft_mbar_wait(bar(FT_B_XCH + 8 + (warp & 3)), 0)) { sx_set_status(status, 9); ok = false; }
    l += xch[(4 + (hf ^ 1)) * FT_BM + r];
    if (ok && !ft_mbar_wait(bar(FT_B_PVDONE), (nb - 1) & 1)) { sx_set_status(status, 8); ok = false; }
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + ((size_t)(t_begin + q0 + r) * nh + h) * FT_HD + hf * FT_HALF;
#pragma unroll 1
      for (int c = 0; c < FT_HALF / 32; ++c) {
        float o[32];
        ft_ld32(t_row + FT_COL_O + hf * FT_HALF + c * 32, o);
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = ft_pack(o[8 * i] * inv, o[8 * i + 1] * inv);
            v.y = ft_pack(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            v.z = ft_pack(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            v.w = ft_pack(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            reinterpret_cast<uint4*>(dst + c * 32)[i] = v;
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == FT_MMA_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)FT_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*ft_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static ft_encode_fn ft_get_encode() {
  static ft_encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = (ft_encode_fn)p;
  }
  return fn;
}

// q [T, nh * 128]: boxes of 128 rows x 64 values
static int ft_map_q(CUtensorMap* map, const void* q, long long T, int nh) {
  ft_encode_fn enc = ft_get_encode();
  if (!enc) return SX_ERR_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)nh * FT_HD, (cuuint64_t)T};
  cuuint64_t strides[1] = {(cuuint64_t)nh * FT_HD * 2};
  cuuint32_t box[2] = {64, FT_BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}
// cache pages [n_pages, nkv, 64, 128]: boxes of one page's 64 tokens x 64 values of one kv head
static int ft_map_pages(CUtensorMap* map, const void* pages, long long n_pages, int nkv) {
  ft_encode_fn enc = ft_get_encode();
  if (!enc) return SX_ERR_SIZE;
  cuuint64_t dims[4] = {FT_HD, SX_PAGE, (cuuint64_t)nkv, (cuuint64_t)n_pages};
  cuuint64_t strides[3] = {FT_HD * 2, (cuuint64_t)SX_PAGE * FT_HD * 2, (cuuint64_t)nkv * SX_PAGE * FT_HD * 2};
  cuuint32_t box[4] = {64, SX_PAGE, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pages), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 20000 + (int)r;
}

static int* ft_status_word() {
  static int* p = nullptr;
  if (!p) p = sx_status_word_alloc();
  return p;
}

// q [T, nh, 128] packed tokens, out [T, nh * 128]; tile_seq/tile_q0 [n_tiles] list 128-row query tiles of the
// sequences; the cache already holds this step's keys and values.  Head size 128 only (SX_ERR_SIZE otherwise).
extern "C" int sx_attn_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out, long long T,
                                  long long n_pages, const int* tile_seq, const int* tile_q0, int n_tiles,
                                  const int* cu_seqlens, const int* seq_past, const int* seq_lens, const int* block_table,
                                  int maxp, int nh, int nkv, int hd, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (hd != FT_HD || nkv <= 0 || nh % nkv != 0 || n_tiles > 65535 || T <= 0 || n_pages <= 0) return SX_ERR_SIZE;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15)) return SX_ERR_ALIGN;
  int* status = ft_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  CUtensorMap mq, mk, mv;
  int rc = ft_map_q(&mq, q, T, nh);
  if (rc) return rc;
  if ((rc = ft_map_pages(&mk, k_pages, n_pages, nkv))) return rc;
  if ((rc = ft_map_pages(&mv, v_pages, n_pages, nkv))) return rc;
  const size_t smem = 1024 + FT_SMEM_TILES + FT_NBARS * sizeof(uint64_t) + 16 + 6 * FT_BM * sizeof(float);
  auto kern = attn_tc_prefill_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return sx_launch(kern, dim3(nh, n_tiles), dim3(FT_THREADS), smem, stream, mq, mk, mv, (bf16*)out, tile_seq, tile_q0,
                   cu_seqlens, seq_past, seq_lens, block_table, maxp, nh, nkv, scale * 1.4426950408889634f, window, status);
}

// 0, or which bounded wait ran out (1 producer, 2-5 MMA issuer, 6-9 softmax)
// Reads the word in host memory: no device call.  It tells of kernels the host has already waited for.
// With reset != 0 the word goes back to 0.
extern "C" int sx_attn_tc_status(int* host_value, int reset) {
  int* p = ft_status_word();
  if (!p) return (int)cudaErrorMemoryAllocation;
  *host_value = *(volatile int*)p;
  if (reset) *(volatile int*)p = 0;
  return 0;
}
