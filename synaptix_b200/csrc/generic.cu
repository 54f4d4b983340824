// Plain kernels for every operation of a decoder step, for float32 and bfloat16 storage,
// all arithmetic in 32-bit (FFMA only: no tensor cores, no TF32).  They take every size;
// they are the whole of the float32 path, and the fallback of the bfloat16 path for sizes
// that the fast kernels refuse.
//
// What they compute follows the reference's formulas:
//   embedding   crates/synaptix-kernels-cuda/src/cu/embed/embed.cu:18-46
//   RMSNorm     crates/synaptix-kernels-cuda/src/cu/reduction/rms_norm.cu:26-98 (plain gain w)
//   residual    crates/synaptix-kernels-cuda/src/cu/fused/norm/rmsnorm_residual.cu:97-159
//   rotary      crates/synaptix-kernels-cuda/src/cu/elementwise/rope.cu:27-118 (rotate-half)
//   KV append   crates/synaptix-kernels-cuda/src/cu/elementwise/kv_append.cu:53-78
//   attention   crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_decode.cu:92-205
//   SiLU*mul    crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-52
//   f32 GEMM    crates/synaptix-kernels-cuda/src/best_cu/gemm/gemm_f32.cu:1-69
// but not how: the residual stream is kept in 32-bit, the cache is paged, tokens of
// sequences with unequal lengths are packed into one stream.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// embedding gather: out[t, :] = float(table[ids[t], :]); an id outside the table gives zeros
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;
  const T* row = table + (size_t)(ok ? id : 0) * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}

extern "C" int sx_embed_gather(const void* table, int dt, const int* ids, float* out,
                               int n_tokens, int H, int V, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dt == SX_F32)
    return sx_launch(embed_gather_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, (const float*)table, ids, out, H, V);
  if (dt == SX_BF16)
    return sx_launch(embed_gather_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, (const bf16*)table, ids, out, H, V);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// residual add + RMSNorm.
//   v = h[t] (+ delta[t]);  if write_h: h[t] = v;  y[r] = v * rsqrt(mean(v^2) + eps) * w
// Rows: r = 0..R-1, t = rows ? rows[r] : r.  h and the sum of squares are 32-bit.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const float* __restrict__ w, float eps, T* __restrict__ y,
                                   const int* __restrict__ rows, int H, int write_h) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* hr = h + (size_t)t * H;
  const T* dr = delta ? delta + (size_t)t * H : nullptr;
  T* yr = y + (size_t)r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hr[i];
    if (dr) {
      v += to_f32(dr[i]);
      if (write_h) hr[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hr[i];
    if (dr && !write_h) v += to_f32(dr[i]);
    yr[i] = from_f32<T>(v * inv * w[i]);
  }
}

// the same with the whole row held in registers (one pass over memory, one reduction):
// rows of up to 256 * 4 * VEC4 elements, H a multiple of 4, 16-byte aligned rows
template <typename T, int VEC4>
__global__ void __launch_bounds__(256) add_rmsnorm_reg_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                                              const float* __restrict__ w, float eps, T* __restrict__ y,
                                                              const int* __restrict__ rows, int H, int write_h) {
  __shared__ float red[33];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float4* hr = reinterpret_cast<float4*>(h + (size_t)t * H);
  const T* dr = delta ? delta + (size_t)t * H : nullptr;
  const int n4 = H >> 2;
  float4 v[VEC4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC4; ++k) {
    const int i = threadIdx.x + k * 256;
    v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n4) {
      v[k] = hr[i];
      if (dr) {
        v[k].x += to_f32(dr[4 * i]); v[k].y += to_f32(dr[4 * i + 1]);
        v[k].z += to_f32(dr[4 * i + 2]); v[k].w += to_f32(dr[4 * i + 3]);
        if (write_h) hr[i] = v[k];
      }
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* yr = y + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < VEC4; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 g = reinterpret_cast<const float4*>(w)[i];
      yr[4 * i] = from_f32<T>(v[k].x * inv * g.x);
      yr[4 * i + 1] = from_f32<T>(v[k].y * inv * g.y);
      yr[4 * i + 2] = from_f32<T>(v[k].z * inv * g.z);
      yr[4 * i + 3] = from_f32<T>(v[k].w * inv * g.w);
    }
  }
}

template <typename T>
static int add_rmsnorm_launch(float* h, const void* delta, const float* w, float eps, void* y, const int* rows, int R,
                              int H, int write_h, cudaStream_t stream) {
  const bool aligned = (H % 4 == 0) && (((uintptr_t)h | (uintptr_t)w) % 16 == 0);
  if (aligned && H <= 256 * 4 * 4)
    return sx_launch(add_rmsnorm_reg_kernel<T, 4>, dim3(R), dim3(256), 0, stream, h, (const T*)delta, w, eps, (T*)y, rows, H, write_h);
  if (aligned && H <= 256 * 4 * 8)
    return sx_launch(add_rmsnorm_reg_kernel<T, 8>, dim3(R), dim3(256), 0, stream, h, (const T*)delta, w, eps, (T*)y, rows, H, write_h);
  return sx_launch(add_rmsnorm_kernel<T>, dim3(R), dim3(256), 0, stream, h, (const T*)delta, w, eps, (T*)y, rows, H, write_h);
}

extern "C" int sx_add_rmsnorm(float* h, const void* delta, const float* w, float eps, void* y,
                              const int* rows, int R, int H, int dt, int write_h,
                              cudaStream_t stream) {
  if (R <= 0) return 0;
  if (dt == SX_F32) return add_rmsnorm_launch<float>(h, delta, w, eps, y, rows, R, H, write_h, stream);
  if (dt == SX_BF16) return add_rmsnorm_launch<bf16>(h, delta, w, eps, y, rows, R, H, write_h, stream);
  return SX_ERR_DTYPE;
}

// h[t] += delta[t] (32-bit residual sum), for the places where no norm follows
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] += to_f32(delta[i]);
}
extern "C" int sx_residual_add(float* h, const void* delta, long long n, int dt, cudaStream_t stream) {
  if (n <= 0) return 0;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dt == SX_F32) residual_add_kernel<float><<<grid, 256, 0, stream>>>(h, (const float*)delta, (size_t)n);
  else if (dt == SX_BF16) residual_add_kernel<bf16><<<grid, 256, 0, stream>>>(h, (const bf16*)delta, (size_t)n);
  else return SX_ERR_DTYPE;
  return sx_launch_status();
}

// ---------------------------------------------------------------------------------------
// C[M,N] = A[M,K] * W[N,K]^T, 32-bit accumulation in k order.  Two kernels:
//   gemm_tile: 64x64x16 tiles, 4x4 outputs per thread (any M);
//   gemm_rows: one warp per output column, up to 8 rows of A at a time (M <= 16).
// ---------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_tile_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        TC* __restrict__ C, int M, int N, int K) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx >> 4, c = idx & 15;
      const int k = k0 + c;
      const int m = m0 + r, n = n0 + r;
      As[c][r] = (m < M && k < K) ? to_f32(A[(size_t)m * K + k]) : 0.f;
      Ws[c][r] = (n < N && k < K) ? to_f32(W[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * N + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(128) gemm_rows_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        TC* __restrict__ C, int M, int N, int K) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (n >= N) return;
  const TW* wr = W + (size_t)n * K;
  for (int m0 = 0; m0 < M; m0 += 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float w = to_f32(wr[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (m0 + i < M) acc[i] = fmaf(to_f32(A[(size_t)(m0 + i) * K + k]), w, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = warp_sum(acc[i]);
      if (lane == 0 && m0 + i < M) C[(size_t)(m0 + i) * N + n] = from_f32<TC>(s);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int gemm_generic_launch(const void* A, const void* W, void* C, int M, int N, int K,
                               cudaStream_t stream) {
  if (M <= 16) {
    gemm_rows_kernel<TA, TW, TC><<<(N + 3) / 4, 128, 0, stream>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    gemm_tile_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K);
  }
  return sx_launch_status();
}

extern "C" int sx_gemm_generic(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt,
                               int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return SX_ERR_SIZE;
  if ((size_t)((M + 63) / 64) > 65535) return SX_ERR_SIZE;
  if (a_dt == SX_F32 && w_dt == SX_F32 && c_dt == SX_F32)
    return gemm_generic_launch<float, float, float>(A, W, C, M, N, K, stream);
  if (a_dt == SX_BF16 && w_dt == SX_BF16 && c_dt == SX_BF16)
    return gemm_generic_launch<bf16, bf16, bf16>(A, W, C, M, N, K, stream);
  if (a_dt == SX_BF16 && w_dt == SX_BF16 && c_dt == SX_F32)
    return gemm_generic_launch<bf16, bf16, float>(A, W, C, M, N, K, stream);
  if (a_dt == SX_F32 && w_dt == SX_BF16 && c_dt == SX_F32)
    return gemm_generic_launch<float, bf16, float>(A, W, C, M, N, K, stream);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// head preparation and cache write, one block per (token, head of the fused projection):
//   q heads: optional RMSNorm over the head (gain wq), optional rotate-half rotation of the
//            first rotary_dim elements by angle pos * inv_freq[i], written to q_out[t, head, :];
//   k heads: the same with wk, written into the sequence's page at the token's position;
//   v heads: copied into the page.
// qkv is [T, (nh + 2 nkv) * hd]: q heads, then k heads, then v heads.
// ---------------------------------------------------------------------------------------
// One block per token, one warp per head at a time.  A lane owns the rotation pairs
// (p, p + rotary_dim/2) for p = lane, lane + 32, ...; their angles, sines and cosines are computed
// once per token and reused for every q and k head.
#define QP_WARPS 8
#define QP_MAXP 8            // pairs per lane: head sizes up to 512
// PP: rotation pairs a lane owns (rotary_dim / 2 <= 32 * PP); angles, sines, cosines and the norm
// gains of its pairs stay in registers for all heads of the token
template <typename T, int PP>
__global__ void __launch_bounds__(QP_WARPS * 32) qkv_prepare_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const float* __restrict__ wq, const float* __restrict__ wk, const float* __restrict__ inv_freq,
    int rotary_dim, float eps, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int maxp, int nh, int nkv, int hd, int n_pages) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int row = (nh + 2 * nkv) * hd;
  const T* src_tok = qkv + (size_t)t * row;
  const int half = inv_freq ? rotary_dim / 2 : 0;

  float cs[PP], sn[PP], gq1[PP], gq2[PP], gk1[PP], gk2[PP];
#pragma unroll
  for (int k = 0; k < PP; ++k) {
    const int p = lane + 32 * k;
    cs[k] = 1.f; sn[k] = 0.f;
    gq1[k] = gq2[k] = gk1[k] = gk2[k] = 1.f;
    if (p < half) {
      sincosf((float)pos * inv_freq[p], &sn[k], &cs[k]);
      if (wq) { gq1[k] = wq[p]; gq2[k] = wq[p + half]; }
      if (wk) { gk1[k] = wk[p]; gk2[k] = wk[p + half]; }
    }
  }
  // where this token's keys and values go
  const int s = seq_of_token[t];
  const int page = block_table[(size_t)s * maxp + (pos >> 6)];
  const bool page_ok = page >= 0 && page < n_pages;     // the host guarantees a page; never write outside
  const bool vec_copy = (hd % 8 == 0) && sizeof(T) == 2;

  for (int head = blockIdx.y * QP_WARPS + warp; head < nh + 2 * nkv; head += gridDim.y * QP_WARPS) {
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);
    const T* src = src_tok + (size_t)head * hd;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nh + head) * hd;
    } else {
      T* base = is_k ? k_pages : v_pages;
      if (!base || !page_ok) continue;                   // a layer that reads another layer's cache writes nothing
      dst = base + (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * hd;
    }
    if (!is_q && !is_k) {                                // v: copy
      if (vec_copy) {
        for (int i = lane; i < hd / 8; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
      } else {
        for (int i = lane; i < hd; i += 32) dst[i] = src[i];
      }
      continue;
    }
    const float* w = is_q ? wq : wk;
    float x1[PP], x2[PP];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PP; ++k) {
      const int p = lane + 32 * k;
      x1[k] = x2[k] = 0.f;
      if (p < half) {
        x1[k] = to_f32(src[p]);
        x2[k] = to_f32(src[p + half]);
        ss += x1[k] * x1[k] + x2[k] * x2[k];
      }
    }
    for (int i = 2 * half + lane; i < hd; i += 32) {     // elements that are not rotated
      const float v = to_f32(src[i]);
      ss += v * v;
    }
    float inv = 1.f;
    if (w) inv = rsqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int k = 0; k < PP; ++k) {
      const int p = lane + 32 * k;
      if (p < half) {
        const float a = x1[k] * inv * (is_q ? gq1[k] : gk1[k]);
        const float b = x2[k] * inv * (is_q ? gq2[k] : gk2[k]);
        dst[p] = from_f32<T>(a * cs[k] - b * sn[k]);
        dst[p + half] = from_f32<T>(a * sn[k] + b * cs[k]);
      }
    }
    for (int i = 2 * half + lane; i < hd; i += 32) {
      const float v = to_f32(src[i]);
      dst[i] = from_f32<T>(w ? v * inv * w[i] : v);
    }
  }
}

// The common case (the whole head is rotated, head size a multiple of 4) with two adjacent pairs per
// lane and iteration, so that every access is 4 bytes (bfloat16) or 8 bytes (float) wide:
// a lane owns pairs p = 64 k + 2 lane + {0, 1}.
template <typename T> struct qp_vec2;
template <> struct qp_vec2<bf16> {
  static __device__ __forceinline__ float2 load(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  static __device__ __forceinline__ void store(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
};
template <> struct qp_vec2<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};

template <typename T, int PQ>
__global__ void __launch_bounds__(QP_WARPS * 32) qkv_prepare_vec_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const float* __restrict__ wq, const float* __restrict__ wk, const float* __restrict__ inv_freq, float eps,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int maxp, int nh, int nkv, int hd, int n_pages) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int row = (nh + 2 * nkv) * hd;
  const T* src_tok = qkv + (size_t)t * row;
  const int half = hd / 2;

  float cs[PQ][2], sn[PQ][2], gq1[PQ][2], gq2[PQ][2], gk1[PQ][2], gk2[PQ][2];
#pragma unroll
  for (int k = 0; k < PQ; ++k)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int p = 64 * k + 2 * lane + j;
      cs[k][j] = 1.f; sn[k][j] = 0.f;
      gq1[k][j] = gq2[k][j] = gk1[k][j] = gk2[k][j] = 1.f;
      if (p < half) {
        if (inv_freq) sincosf((float)pos * inv_freq[p], &sn[k][j], &cs[k][j]);
        if (wq) { gq1[k][j] = wq[p]; gq2[k][j] = wq[p + half]; }
        if (wk) { gk1[k][j] = wk[p]; gk2[k][j] = wk[p + half]; }
      }
    }
  const int s = seq_of_token[t];
  const int page = block_table[(size_t)s * maxp + (pos >> 6)];
  const bool page_ok = page >= 0 && page < n_pages;

  for (int head = blockIdx.y * QP_WARPS + warp; head < nh + 2 * nkv; head += gridDim.y * QP_WARPS) {
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);
    const T* src = src_tok + (size_t)head * hd;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nh + head) * hd;
    } else {
      T* base = is_k ? k_pages : v_pages;
      if (!base || !page_ok) continue;
      dst = base + (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * hd;
    }
    if (!is_q && !is_k) {                                // v: copy, 4 elements a lane and round
      for (int i = lane * 4; i < hd; i += 128) {
        const float2 a = qp_vec2<T>::load(src + i), b = qp_vec2<T>::load(src + i + 2);
        qp_vec2<T>::store(dst + i, a.x, a.y);
        qp_vec2<T>::store(dst + i + 2, b.x, b.y);
      }
      continue;
    }
    const bool normed = (is_q ? wq : wk) != nullptr;
    float2 x1[PQ], x2[PQ];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < PQ; ++k) {
      const int p = 64 * k + 2 * lane;
      x1[k] = x2[k] = make_float2(0.f, 0.f);
      if (p < half) {
        x1[k] = qp_vec2<T>::load(src + p);
        x2[k] = qp_vec2<T>::load(src + p + half);
        ss += x1[k].x * x1[k].x + x1[k].y * x1[k].y + x2[k].x * x2[k].x + x2[k].y * x2[k].y;
      }
    }
    float inv = 1.f;
    if (normed) inv = rsqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int k = 0; k < PQ; ++k) {
      const int p = 64 * k + 2 * lane;
      if (p < half) {
        const float a0 = x1[k].x * inv * (is_q ? gq1[k][0] : gk1[k][0]), a1 = x1[k].y * inv * (is_q ? gq1[k][1] : gk1[k][1]);
        const float b0 = x2[k].x * inv * (is_q ? gq2[k][0] : gk2[k][0]), b1 = x2[k].y * inv * (is_q ? gq2[k][1] : gk2[k][1]);
        qp_vec2<T>::store(dst + p, a0 * cs[k][0] - b0 * sn[k][0], a1 * cs[k][1] - b1 * sn[k][1]);
        qp_vec2<T>::store(dst + p + half, a0 * sn[k][0] + b0 * cs[k][0], a1 * sn[k][1] + b1 * cs[k][1]);
      }
    }
  }
}

// bfloat16, the whole head rotated (or nothing), head size 64 or 128, many tokens: 16 values a lane (8 from
// each half of the head, two 16-byte loads), so HD/16 lanes share a head and a warp works on 32/(HD/16) heads
// at once; sines, cosines and gains are computed once per block into shared memory.  The kernel above spends
// ~25 instructions per value (4 values a lane, every warp recomputing the token's sines): measured 24 us for
// 2,048 tokens x 48 heads, bound by instruction issue, where memory alone would need 8.
template <int HD>
__global__ void __launch_bounds__(QP_WARPS * 32) qkv_prepare_wide_kernel(
    const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
    const float* __restrict__ wq, const float* __restrict__ wk, const float* __restrict__ inv_freq, float eps,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int maxp, int nh, int nkv, int n_pages) {
  constexpr int HALF = HD / 2, LPH = HD / 16, HPW = 32 / LPH;      // lanes a head, heads a warp
  __shared__ float s_cs[HALF], s_sn[HALF], s_gq[HD], s_gk[HD];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < HALF; i += QP_WARPS * 32) {
    float sn = 0.f, cs = 1.f;
    if (inv_freq) sincosf((float)pos * inv_freq[i], &sn, &cs);
    s_cs[i] = cs;
    s_sn[i] = sn;
  }
  for (int i = threadIdx.x; i < HD; i += QP_WARPS * 32) {
    s_gq[i] = wq ? wq[i] : 1.f;
    s_gk[i] = wk ? wk[i] : 1.f;
  }
  const int s = seq_of_token[t];
  const int page = block_table[(size_t)s * maxp + (pos >> 6)];
  const bool page_ok = page >= 0 && page < n_pages;
  __syncthreads();

  const int n_heads = nh + 2 * nkv;
  const bf16* src_tok = qkv + (size_t)t * n_heads * HD;
  const int sub = lane / LPH, e0 = (lane % LPH) * 8;               // which head of the warp's group; first value
  for (int hg = (blockIdx.y * QP_WARPS + warp) * HPW; hg < n_heads; hg += gridDim.y * QP_WARPS * HPW) {
    const int head = hg + sub;
    const bool live = head < n_heads;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (live) {
      const bf16* src = src_tok + (size_t)head * HD + e0;
      a = *reinterpret_cast<const uint4*>(src);
      b = *reinterpret_cast<const uint4*>(src + HALF);
    }
    bf16* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = q_out + ((size_t)t * nh + head) * HD + e0;
      } else {
        bf16* base = is_k ? k_pages : v_pages;
        const int kvh = is_k ? head - nh : head - nh - nkv;
        if (base && page_ok) dst = base + (((size_t)page * nkv + kvh) * SX_PAGE + (pos & 63)) * HD + e0;
      }
    }
    float x1[8], x2[8];
    const uint32_t* au = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* bu = reinterpret_cast<const uint32_t*>(&b);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&au[i]));
      const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bu[i]));
      x1[2 * i] = fa.x; x1[2 * i + 1] = fa.y; x2[2 * i] = fb.x; x2[2 * i + 1] = fb.y;
      ss += fa.x * fa.x + fa.y * fa.y + fb.x * fb.x + fb.y * fb.y;
    }
    // the head's sum of squares over its LPH lanes (every lane takes part; v heads carry theirs along unused)
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!dst) continue;
    if (is_q || is_k) {
      const float* gn = is_q ? s_gq : s_gk;
      const bool normed = (is_q ? wq : wk) != nullptr;
      const float inv = normed ? rsqrtf(ss / (float)HD + eps) : 1.f;
      uint32_t* ao = reinterpret_cast<uint32_t*>(&a);
      uint32_t* bo = reinterpret_cast<uint32_t*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float lo[2], hi[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int e = e0 + 2 * i + j;
          const float u = x1[2 * i + j] * inv * gn[e], w = x2[2 * i + j] * inv * gn[e + HALF];
          lo[j] = u * s_cs[e] - w * s_sn[e];
          hi[j] = u * s_sn[e] + w * s_cs[e];
        }
        __nv_bfloat162 plo = __floats2bfloat162_rn(lo[0], lo[1]), phi = __floats2bfloat162_rn(hi[0], hi[1]);
        ao[i] = *reinterpret_cast<uint32_t*>(&plo);
        bo[i] = *reinterpret_cast<uint32_t*>(&phi);
      }
    }
    *reinterpret_cast<uint4*>(dst) = a;
    *reinterpret_cast<uint4*>(dst + HALF) = b;
  }
}

template <typename T>
static int qkv_prepare_launch(dim3 grid, cudaStream_t stream, const void* qkv, void* q_out, void* k_pages, void* v_pages,
                              const float* wq, const float* wk, const float* inv_freq, int rotary_dim, float eps,
                              const int* positions, const int* seq_of_token, const int* block_table, int maxp, int nh,
                              int nkv, int hd, int n_pages) {
  const int pairs = inv_freq ? rotary_dim / 2 : 0;
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 7) == 0;
  if (sizeof(T) == 2 && (hd == 128 || hd == 64) && (!inv_freq || rotary_dim == hd) && grid.y == 1 &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0) {
#define QP_WGO(HD)                                                                                                       \
  return sx_launch(qkv_prepare_wide_kernel<HD>, grid, dim3(QP_WARPS * 32), 0, stream, (const bf16*)qkv, (bf16*)q_out,      \
                   (bf16*)k_pages, (bf16*)v_pages, wq, wk, inv_freq, eps, positions, seq_of_token, block_table, maxp, nh,  \
                   nkv, n_pages)
    if (hd == 128) QP_WGO(128);
    QP_WGO(64);
#undef QP_WGO
  }
  if (hd % 4 == 0 && hd <= 512 && aligned && (!inv_freq || rotary_dim == hd)) {
#define QP_VGO(PQ)                                                                                                     \
  return sx_launch(qkv_prepare_vec_kernel<T, PQ>, grid, dim3(QP_WARPS * 32), 0, stream, (const T*)qkv, (T*)q_out, (T*)k_pages, \
                   (T*)v_pages, wq, wk, inv_freq, eps, positions, seq_of_token, block_table, maxp, nh, nkv, hd, n_pages)
    if (hd <= 128) QP_VGO(1);
    else if (hd <= 256) QP_VGO(2);
    else QP_VGO(4);
#undef QP_VGO
  }
#define QP_GO(PP)                                                                                                   \
  return sx_launch(qkv_prepare_kernel<T, PP>, grid, dim3(QP_WARPS * 32), 0, stream, (const T*)qkv, (T*)q_out, (T*)k_pages, \
                   (T*)v_pages, wq, wk, inv_freq, rotary_dim, eps, positions, seq_of_token, block_table, maxp, nh, nkv, hd, n_pages)
  if (pairs <= 32) QP_GO(1);
  else if (pairs <= 64) QP_GO(2);
  else if (pairs <= 128) QP_GO(4);
  else QP_GO(8);
#undef QP_GO
}

extern "C" int sx_qkv_prepare(const void* qkv, void* q_out, void* k_pages, void* v_pages,
                              const float* wq, const float* wk, const float* inv_freq, int rotary_dim,
                              float eps, const int* positions, const int* seq_of_token,
                              const int* block_table, int maxp, int n_tokens, int nh, int nkv, int hd,
                              int n_pages, int dt, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || (rotary_dim & 1) || rotary_dim > hd || rotary_dim / 2 > 32 * QP_MAXP) return SX_ERR_SIZE;
  // few tokens: spread the heads over blocks too, so that the step is one round of work
  const int heads = nh + 2 * nkv;
  dim3 grid(n_tokens, n_tokens <= 64 ? (heads + QP_WARPS - 1) / QP_WARPS : 1);
  if (dt == SX_F32)
    return qkv_prepare_launch<float>(grid, stream, qkv, q_out, k_pages, v_pages, wq, wk, inv_freq, rotary_dim, eps, positions,
                                     seq_of_token, block_table, maxp, nh, nkv, hd, n_pages);
  if (dt == SX_BF16)
    return qkv_prepare_launch<bf16>(grid, stream, qkv, q_out, k_pages, v_pages, wq, wk, inv_freq, rotary_dim, eps, positions,
                                    seq_of_token, block_table, maxp, nh, nkv, hd, n_pages);
  return SX_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------
// cosines and sines of position * inv_freq[i] for every token of a step, [n_tokens, pairs] each: what the head
// preparation computes per token, made once for a product whose epilogue prepares the heads
// ---------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int pairs,
                                  float* __restrict__ cs, float* __restrict__ sn, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / pairs;
  const int i = (int)(idx - t * pairs);
  float s, c;
  sincosf((float)positions[t] * inv_freq[i], &s, &c);
  cs[idx] = c;
  sn[idx] = s;
}
extern "C" int sx_rope_table(const int* positions, const float* inv_freq, int pairs, int n_tokens, float* cs, float* sn,
                             cudaStream_t stream) {
  if (n_tokens <= 0 || pairs <= 0) return 0;
  const size_t n = (size_t)n_tokens * pairs;
  return sx_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, positions, inv_freq, pairs, cs, sn, n);
}

// ---------------------------------------------------------------------------------------
// attention over the paged cache, one block per (token, query head): scores of the keys
// lo..pos in tiles of 128, running maximum and sum (online softmax), all in 32-bit.
//   lo = window > 0 ? max(0, pos - window + 1) : 0;  query head h reads kv head h / (nh/nkv).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) attn_generic_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int maxp, int nh, int nkv, int hd, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;            // hd
  float* ps = smem + hd;       // 128
  __shared__ float red[33];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)seq_of_token[t] * maxp;
  const int kvh = h / (nh / nkv);
  const T* qr = q + ((size_t)t * nh + h) * hd;
  for (int i = tid; i < hd; i += 128) qs[i] = to_f32(qr[i]);
  __syncthreads();

  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};     // hd <= 512

  for (int j0 = lo; j0 <= pos; j0 += 128) {
    const int j = j0 + tid;
    float s = -INFINITY;
    if (j <= pos) {
      const int page = bt[j >> 6];
      const T* kr = k_pages + (((size_t)page * nkv + kvh) * SX_PAGE + (j & 63)) * hd;
      float d = 0.f;
      for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
      s = d * scale;
    }
    const float tmax = block_max(s, red);
    const float m_new = fmaxf(m, tmax);
    const float p = (j <= pos) ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    ps[tid] = p;
    const float psum = block_sum(p, red);   // also orders the writes to ps before the reads below
    l = l * corr + psum;
    const int ntile = min(128, pos - j0 + 1);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int d = tid + a * 128;
      if (d < hd) {
        float v = acc[a] * corr;
        for (int jj = 0; jj < ntile; ++jj) {
          const int jk = j0 + jj;
          const int page = bt[jk >> 6];
          v = fmaf(ps[jj], to_f32(v_pages[(((size_t)page * nkv + kvh) * SX_PAGE + (jk & 63)) * hd + d]), v);
        }
        acc[a] = v;
      }
    }
    m = m_new;
    __syncthreads();
  }
  T* o = out + ((size_t)t * nh + h) * hd;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int d = tid + a * 128;
    if (d < hd) o[d] = from_f32<T>(acc[a] / l);
  }
}

extern "C" int sx_attn_generic(const void* q, const void* k_pages, const void* v_pages, void* out,
                               const int* positions, const int* seq_of_token, const int* block_table,
                               int maxp, int n_tokens, int nh, int nkv, int hd, float scale, int window,
                               int dt, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || hd > 512 || nkv <= 0 || nh % nkv != 0 || nh > 65535) return SX_ERR_SIZE;
  dim3 grid(n_tokens, nh);
  const size_t smem = (size_t)(hd + 128) * sizeof(float);
  if (dt == SX_F32)
    attn_generic_kernel<float><<<grid, 128, smem, stream>>>(
        (const float*)q, (const float*)k_pages, (const float*)v_pages, (float*)out, positions, seq_of_token,
        block_table, maxp, nh, nkv, hd, scale, window);
  else if (dt == SX_BF16)
    attn_generic_kernel<bf16><<<grid, 128, smem, stream>>>(
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, positions, seq_of_token,
        block_table, maxp, nh, nkv, hd, scale, window);
  else
    return SX_ERR_DTYPE;
  return sx_launch_status();
}

// ---------------------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(x) = x / (1 + exp(-x)), in 32-bit
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t n) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = to_f32(gu[t * 2 * I + i]);
  const float u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

extern "C" int sx_silu_mul(const void* gu, void* out, int n_tokens, int I, int dt, cudaStream_t stream) {
  const size_t n = (size_t)n_tokens * I;
  if (n == 0) return 0;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dt == SX_F32) silu_mul_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)out, I, n);
  else if (dt == SX_BF16) silu_mul_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gu, (bf16*)out, I, n);
  else return SX_ERR_DTYPE;
  return sx_launch_status();
}

// ---------------------------------------------------------------------------------------
// Decoding that stays on the device.  Before a step: a row whose control word is not negative
// runs that token instead of the one sampled for it in the step before (and its history of
// tokens, if kept for the penalties, ends with that token).  After a step: every live row
// (advance_by = 1) takes its sampled token as the next input, appends it to its history, and
// moves one position and one word of its random stream on; rows that pad the batch stay put.
// ---------------------------------------------------------------------------------------
__global__ void decode_begin_kernel(int* __restrict__ token_ids, const int* __restrict__ control,
                                    int* __restrict__ history, const int* __restrict__ hist_len, int hist_cap, int S) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  const int t = control[i];
  if (t < 0) return;
  token_ids[i] = t;
  if (history != nullptr) {
    const int n = hist_len[i];
    if (n > 0 && n <= hist_cap) history[(size_t)i * hist_cap + n - 1] = t;
  }
}
extern "C" int sx_decode_begin(int* token_ids, const int* control, int* history, const int* hist_len, int hist_cap,
                               int S, cudaStream_t stream) {
  if (S <= 0) return 0;
  return sx_launch(decode_begin_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, token_ids, control, history,
                   hist_len, hist_cap, S);
}

__global__ void decode_advance_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                      int* __restrict__ positions, int* __restrict__ seq_past,
                                      int* __restrict__ seq_lens, int* __restrict__ rng_step,
                                      const int* __restrict__ advance_by, int* __restrict__ history,
                                      int* __restrict__ hist_len, int hist_cap, int S) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  const int by = advance_by != nullptr ? advance_by[i] : 1;
  if (by == 0) return;
  const int t = sampled[i];
  token_ids[i] = t;
  positions[i] += 1;
  seq_past[i] += 1;
  seq_lens[i] += 1;
  if (rng_step != nullptr) rng_step[i] += 1;
  if (history != nullptr) {
    const int n = hist_len[i];
    if (n < hist_cap) {
      history[(size_t)i * hist_cap + n] = t;
      hist_len[i] = n + 1;
    }
  }
}
extern "C" int sx_decode_advance(int* token_ids, const int* sampled, int* positions, int* seq_past, int* seq_lens,
                                 int* rng_step, const int* advance_by, int* history, int* hist_len, int hist_cap,
                                 int S, cudaStream_t stream) {
  if (S <= 0) return 0;
  return sx_launch(decode_advance_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, token_ids, sampled, positions,
                   seq_past, seq_lens, rng_step, advance_by, history, hist_len, hist_cap, S);
}
