// Shared helpers for the sm_100a kernels: error reporting, vector loads, reductions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/dejavu_b200.h"

namespace djv {

// ---- host side ----------------------------------------------------------------------------
void set_error(const char *fmt, ...);
void count_launch(int n = 1);
int check_launch(const char *what);  // cudaGetLastError -> status

#define DJV_REQUIRE(cond, ...)          \
  do {                                  \
    if (!(cond)) {                      \
      djv::set_error(__VA_ARGS__);      \
      return DJV_ERR_INVALID;           \
    }                                   \
  } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
int sm_count();  // multiprocessors of the current device (cached per device)
// integer development knob from the environment (callers read it once into a static)
inline int env_int(const char *name, int dflt) {
  const char *v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}

// Kernel launch with programmatic dependent launch (PDL): the next kernel of a stream may be scheduled
// while this one is still running; every kernel of this library starts with pdl_prologue(), which (1) lets
// its own successor be scheduled early and (2) waits until all its predecessors have completed and their
// writes are visible, before it touches any memory. Only launch latency is overlapped; ordering of data is
// the same as without PDL. DJV_PDL=0 in the environment launches the classic way.
bool pdl_enabled();
// Set by djv_set_early_weight_prefetch for the calling thread: kernels may read their index list / attention
// state and prefetch weight rows into L2 before they wait for the kernel launched just before them.
bool early_prefetch();

template <typename... P, typename... A>
inline cudaError_t launch_kernel(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 A &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// The same with thread-block clusters of `cluster` blocks (for kernels without compile-time cluster dims).
template <typename... P, typename... A>
inline cudaError_t launch_kernel_cluster(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                         dim3 cluster, A &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// ---- device side --------------------------------------------------------------------------
constexpr int WARP = 32;

__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Hint: bring the 128-byte line at p into L2 (fire and forget).
__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// 16-byte read-only load that does not pollute L1 (weights are streamed exactly once).
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Pins a loaded value at this point of the instruction stream: placed after a group of ld_stream16 calls (all
// of them volatile asm, hence kept in order), it keeps the compiler from sinking the later loads of the group
// below arithmetic on the earlier ones, i.e. all loads of the group are in flight before any is consumed.
__device__ __forceinline__ void keep_loaded(uint4 &v) {
  asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w));
}

// 16-byte cached load (activations, small reused vectors).
__device__ __forceinline__ uint4 ld_cached16(const void *p) {
  return __ldg(reinterpret_cast<const uint4 *>(p));
}

__device__ __forceinline__ float2 h2f(uint32_t u) {
  __half2 h = *reinterpret_cast<__half2 *>(&u);
  return __half22float2(h);
}

// dot of 8 fp16 (packed in a uint4) with 8 fp16 (packed in a uint4), fp32 accumulate
__device__ __forceinline__ float dot8(const uint4 &a, const uint4 &b, float acc) {
  float2 a0 = h2f(a.x), a1 = h2f(a.y), a2 = h2f(a.z), a3 = h2f(a.w);
  float2 b0 = h2f(b.x), b1 = h2f(b.y), b2 = h2f(b.z), b3 = h2f(b.w);
  acc = fmaf(a0.x, b0.x, acc);
  acc = fmaf(a0.y, b0.y, acc);
  acc = fmaf(a1.x, b1.x, acc);
  acc = fmaf(a1.y, b1.y, acc);
  acc = fmaf(a2.x, b2.x, acc);
  acc = fmaf(a2.y, b2.y, acc);
  acc = fmaf(a3.x, b3.x, acc);
  acc = fmaf(a3.y, b3.y, acc);
  return acc;
}

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

template <int ACT>
__device__ __forceinline__ float apply_act(float v) {
  if (ACT == DJV_ACT_RELU) return fmaxf(v, 0.f);
  if (ACT == DJV_ACT_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (ACT == DJV_ACT_GELU_APPROX)
    return 0.5f * v * (1.f + tanhf(0.79788456080286536f * v * (1.f + 0.044715f * v * v)));
  if (ACT == DJV_ACT_SQUARED_RELU) {
    float r = fmaxf(v, 0.f);
    return r * r;
  }
  return v;
}

}  // namespace djv

namespace djv {
// idx == nullptr means the identity index list
__device__ __forceinline__ long long load_index(const void *idx, int m, int idx64) {
  if (idx == nullptr) return m;
  return idx64 ? reinterpret_cast<const long long *>(idx)[m]
               : static_cast<long long>(reinterpret_cast<const int *>(idx)[m]);
}
}  // namespace djv
