// Shared helpers of the sm_100a kernels: element conversion, warp and block
// reductions, and the error channel of the C launchers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

typedef __nv_bfloat16 bf16;

// ---- error channel ---------------------------------------------------------
// Every launcher returns 0 on success.  On a refusal (sizes a kernel does not take)
// or a CUDA launch error it returns non-zero and leaves a message that
// g2b_last_error() of the same shared object returns.
static thread_local char g2b_error_text[512] = "";

#define G2B_REFUSE(...)                                                   \
  do {                                                                    \
    snprintf(g2b_error_text, sizeof(g2b_error_text), __VA_ARGS__);        \
    return 1;                                                             \
  } while (0)

static inline int g2b_check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g2b_error_text, sizeof(g2b_error_text), "%s: %s", what, cudaGetErrorString(e));
    return 2;
  }
  return 0;
}

// Programmatic dependent launch: with the switch on, a kernel is launched with the
// programmatic-stream-serialization attribute, so its blocks may start while the kernel
// before it in the stream is still running.  Every kernel of this library therefore calls
// pdl_wait() before it reads anything an earlier kernel wrote and before its first write,
// and may do independent work (index arithmetic, streaming WEIGHTS into registers) above
// that line; pdl_launch() lets the next kernel start its own independent part.  Both are
// no-ops for a kernel launched the ordinary way.
static int g2b_pdl_enabled = 0;

#define G2B_DEFINE_LAST_ERROR                                            \
  extern "C" const char *g2b_last_error() { return g2b_error_text; }    \
  extern "C" void g2b_set_pdl(int on) { g2b_pdl_enabled = on; }

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// cluster_x > 1 launches thread-block clusters of that many CTAs along x.
template <typename... KArgs, typename... Args>
static inline void g2b_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (g2b_pdl_enabled) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);       // errors surface in g2b_check_launch
}

template <typename... KArgs, typename... Args>
static inline void g2b_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  g2b_launch_cluster(kernel, grid, block, smem, stream, 1u, args...);
}

// What a launcher has to do once per DEVICE (cudaFuncSetAttribute holds for the device that
// is current when it is called, not for the process): `static G2bPerDevice done;` and
//   const int dev = g2b_current_device();
//   if (dev < 0 || !done.value[dev]) { ...set attributes...; if (dev >= 0) done.value[dev] = 1; }
// Two threads that meet in a device's first call both set the attributes; that is harmless.
constexpr int G2B_MAX_DEVICES = 64;
struct G2bPerDevice { int value[G2B_MAX_DEVICES] = {}; };
static inline int g2b_current_device() {
  int d = -1;
  return (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < G2B_MAX_DEVICES) ? d : -1;
}

// element type codes used by the launchers
enum { G2B_F32 = 0, G2B_BF16 = 1 };

// ---- conversion ------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions ------------------------------------------------------------
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

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on the block size.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < n_warps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < n_warps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}
