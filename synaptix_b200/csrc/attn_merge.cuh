// The second kernel of split decode attention: adds up the partial results of a (sequence, query head)'s splits.
// Included by attention.cu and attn_decode.cu.
#pragma once
#include "common.cuh"

// merge of the splits: grid (S * nh), HD threads.  Maxima and sums of all splits are fetched at
// once into shared memory and reduced by one warp; the weighted sum over splits then runs with
// independent loads.
#define AT_MAX_SPLITS 4096      // 32 KB of shared memory in the merge

template <int HD>
__global__ void __launch_bounds__(HD) attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                        bf16* __restrict__ out, int n_splits) {
  extern __shared__ float sm[];                  // m[n_splits] (then weights), l[n_splits]
  float* fac = sm;
  float* ls = sm + n_splits;
  __shared__ float s_L;
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const int d = threadIdx.x;
  // the first splits' outputs are asked for together with the maxima and sums, not after the weights are known
  constexpr int EARLY = 32;
  const float* po = part_o + row * n_splits * HD + d;
  float pv[EARLY];
#pragma unroll
  for (int i = 0; i < EARLY; ++i) pv[i] = i < n_splits ? po[(size_t)i * HD] : 0.f;
  for (int i = d; i < n_splits; i += HD) {
    const float2 ml = reinterpret_cast<const float2*>(part_ml)[row * n_splits + i];
    fac[i] = ml.x;
    ls[i] = ml.y;
  }
  __syncthreads();
  if (d < 32) {
    float M = -INFINITY;
    for (int i = d; i < n_splits; i += 32) M = fmaxf(M, fac[i]);
    M = warp_max(M);
    float L = 0.f;
    for (int i = d; i < n_splits; i += 32) {
      const float mi = fac[i];
      const float f = (mi == -INFINITY) ? 0.f : exp2f(mi - M);
      fac[i] = f;
      L += ls[i] * f;
    }
    // lanes in index order: a fixed order of addition
    L = warp_sum(L);
    if (d == 0) s_L = L;
  }
  __syncthreads();
  float O = 0.f;
#pragma unroll
  for (int i = 0; i < EARLY; ++i) if (i < n_splits) O += pv[i] * fac[i];
#pragma unroll 8
  for (int i = EARLY; i < n_splits; ++i) O += po[(size_t)i * HD] * fac[i];
  const float L = s_L;
  out[row * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

