// Pieces of the tensor-parallel exchange that kernels other than the all-reduce itself use: the comm object,
// and the stores with which a kernel that has just finished part of this rank's partial sum sends it
// straight into every rank's receive buffer (see comm.cu for the protocol). A GEMV kernel that pushes its
// result this way overlaps the NVLink trip with its own tail and with the launch of the all-reduce kernel,
// which then only waits for the pieces, adds them and normalises.
#pragma once
#include "common.cuh"

struct djv_comm {
  int rank, world;
  size_t slot_bytes;
  // device-side tables (cudaMalloc'ed by djv_comm_create)
  void **bufs_dev;
  unsigned *epoch_dev;  // [0] epoch, [1] status
  cudaStream_t last_stream;
};

namespace djv {

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_SLOTS = 3;
constexpr unsigned AR_SENTINEL2 = 0x80008000u;  // two fp16 -0.0

// where a kernel sends its part of the partial sum; bufs == nullptr: nowhere (plain output)
struct PushTarget {
  void *const *bufs;             // device table of every rank's receive buffer
  const unsigned *epoch_status;  // [0] epoch: read-only here, advanced by the all-reduce kernel
  int rank, world;
  size_t slot_bytes;
};

inline PushTarget push_target(const djv_comm *c) {
  PushTarget t{};
  if (c) {
    t.bufs = c->bufs_dev;
    t.epoch_status = c->epoch_dev;
    t.rank = c->rank;
    t.world = c->world;
    t.slot_bytes = c->slot_bytes;
  }
  return t;
}

__device__ __forceinline__ void st_sys16(void *p, const uint4 &v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_sys8(void *p, const uint2 &v) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ uint4 ld_sys16(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// -0.0 halves become +0.0
__device__ __forceinline__ unsigned no_sentinel2(unsigned w) {
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}
__device__ __forceinline__ bool has_sentinel2(unsigned w) {
  return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u;
}
__device__ __forceinline__ bool arrived16(const uint4 &v) {
  return !(has_sentinel2(v.x) || has_sentinel2(v.y) || has_sentinel2(v.z) || has_sentinel2(v.w));
}

// byte offset of piece [rank] of the current slot inside every receive buffer
__device__ __forceinline__ size_t push_piece_offset(const PushTarget &t) {
  const unsigned epoch = t.epoch_status[0];
  return ((size_t)(epoch % AR_SLOTS) * t.world + t.rank) * t.slot_bytes;
}

// 8 (or 4) consecutive fp16 of this rank's partial, element offset `elem` (a multiple of 8 / 4), to every rank
__device__ __forceinline__ void push16(const PushTarget &t, size_t piece_off, size_t elem, uint4 v) {
  v.x = no_sentinel2(v.x); v.y = no_sentinel2(v.y); v.z = no_sentinel2(v.z); v.w = no_sentinel2(v.w);
#pragma unroll
  for (int p = 0; p < AR_MAX_WORLD; ++p)
    if (p < t.world) st_sys16(static_cast<char *>(t.bufs[p]) + piece_off + elem * 2, v);
}
__device__ __forceinline__ void push8(const PushTarget &t, size_t piece_off, size_t elem, uint2 v) {
  v.x = no_sentinel2(v.x); v.y = no_sentinel2(v.y);
#pragma unroll
  for (int p = 0; p < AR_MAX_WORLD; ++p)
    if (p < t.world) st_sys8(static_cast<char *>(t.bufs[p]) + piece_off + elem * 2, v);
}

}  // namespace djv
