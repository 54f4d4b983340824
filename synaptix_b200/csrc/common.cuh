// Shared helpers of the sm_100a kernels: dtype codes, loads/stores with 32-bit math,
// reductions with a fixed order, launch-error reporting.
//
// Every exported function is `extern "C" int sx_*(..., cudaStream_t stream)` and returns
// 0 or a cudaError_t of the launch (never of the kernel's execution: nothing synchronises).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define SX_F32 0
#define SX_BF16 1

// error codes of argument checks (outside cudaError_t's range)
#define SX_ERR_DTYPE 10001
#define SX_ERR_SIZE 10002
#define SX_ERR_ALIGN 10003

typedef __nv_bfloat16 bf16;

template <typename T> struct sx_type;
template <> struct sx_type<float> { static constexpr int code = SX_F32; };
template <> struct sx_type<bf16> { static constexpr int code = SX_BF16; };

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed order (lanes by butterfly, then warps in index order).
// `red` is shared memory of at least 33 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < nwarp; ++i) s += red[i];
    red[32] = s;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = red[0];
    for (int i = 1; i < nwarp; ++i) s = fmaxf(s, red[i]);
    red[32] = s;
  }
  __syncthreads();
  return red[32];
}

static inline int sx_launch_status() { return (int)cudaGetLastError(); }

// ---------------------------------------------------------------------------------------
// Status words of kernels with bounded waits.  A word lives in pinned host memory that the
// device can write (one per library): a kernel whose wait ran out stores a code there, and the
// host reads it without a device call once it has waited for the kernel by any means.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void sx_set_status(int* status, int code) {
  *(volatile int*)status = code;
  __threadfence_system();
}
static inline int* sx_status_word_alloc() {
  int* h = nullptr;
  if (cudaHostAlloc((void**)&h, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return nullptr;
  *h = 0;
  return h;          // unified addressing: the same pointer is valid on the device
}

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through sx_launch may be scheduled while its
// predecessor in the stream is still running.  It must call pdl_wait() before it reads anything
// an earlier kernel wrote or writes anything an earlier kernel may still read; what it does
// before that (asking for its weights) overlaps the predecessor's end.  pdl_trigger() lets the
// NEXT kernel be scheduled; it is called only AFTER pdl_wait(), so that at most one kernel waits
// behind the running one (a kernel that triggered before waiting would let the whole chain of
// later kernels pile up on the SMs, spinning).  Both are no-ops for a kernel launched normally.
// sx_set_pdl(0), exported by every library, turns the launch attribute off for that library.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static int g_sx_pdl = 1;
extern "C" void sx_set_pdl(int on) { g_sx_pdl = on ? 1 : 0; }
static inline bool sx_pdl_enabled() { return g_sx_pdl != 0; }

template <typename... KArgs, typename... Args>
static inline int sx_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = sx_pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// The same launch for a kernel whose blocks form clusters of `cluster` consecutive blocks along x
// (thread-block clusters: the blocks of a cluster run at the same time and may read one another's
// shared memory).  More than 8 blocks a cluster is a size the kernel has to be opted into.
template <typename... KArgs, typename... Args>
static inline int sx_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    int cluster, Args... args) {
  if (cluster > 8) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = sx_pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
// rank of this block in its cluster; a barrier over all threads of the cluster (release / acquire); a load from
// the shared memory of the cluster's block `rank` at the place that `local` names in this block's own
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float cluster_load_f32(const float* local, uint32_t rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(r) : "memory");
  return v;
}

#define SX_PAGE 64
