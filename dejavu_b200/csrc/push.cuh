// Pieces of the tensor-parallel exchange that kernels other than the exchange kernel itself use: the comm
// object, the slot arithmetic, and the stores with which a kernel that has just finished part of this rank's
// partial sum sends it straight into every rank's receive buffer (see exchange.cuh for the protocol). A GEMV
// kernel that pushes its result this way overlaps the NVLink trip with its own tail and with the launch of
// the kernel that consumes the exchange, which then only waits for the pieces, adds them and normalises.
#pragma once
#include "common.cuh"

struct djv_comm {
  int rank, world;
  size_t slot_bytes;
  // device-side tables (cudaMalloc'ed by djv_comm_create)
  void **bufs_dev;
  unsigned *ctl_dev;  // [0] exchanges completed in earlier steps (advanced by djv_comm_end_step), [1] status,
                      // [AR_CTL_EXTENT + slot] bytes per piece the slot's last exchange wrote
  cudaStream_t last_stream;
};

namespace djv {

constexpr int AR_MAX_WORLD = 8;
// Receive slots per rank. Exchange number e (counted since the comm was created) uses slot e % 4. The kernel on
// the main stream that consumes exchange e refills slot (e + 2) % 4 with the sentinel: that slot held exchange
// e - 2, whose readers on this rank are finished (its main consumer precedes this kernel on the stream; a side
// consumer of e - 2 produces something the consumer of e waited for), and no peer writes it again before
// exchange e + 2, which a peer can only start after it has received this rank's piece of e + 1, sent after this
// kernel ended. Slots (e + 1) % 4 and (e + 3) % 4 are left alone: peers may already be filling the first and a
// side stream may still be reading the second.
constexpr int AR_SLOTS = 4;
constexpr int AR_CTL_EXTENT = 4;  // first of the AR_SLOTS per-slot extent records in the control words
constexpr int AR_CTL_WORDS = AR_CTL_EXTENT + AR_SLOTS;
constexpr unsigned AR_SENTINEL2 = 0x80008000u;  // two fp16 -0.0

// where a kernel sends its part of the partial sum; bufs == nullptr: nowhere (plain output)
struct PushTarget {
  void *const *bufs;    // device table of every rank's receive buffer
  const unsigned *ctl;  // [0] exchanges completed in earlier steps: read-only here
  int rank, world;
  size_t slot_bytes;
  int seq;              // number of this exchange inside the current step
};

inline PushTarget push_target(const djv_comm *c, int seq) {
  PushTarget t{};
  if (c) {
    t.bufs = c->bufs_dev;
    t.ctl = c->ctl_dev;
    t.rank = c->rank;
    t.world = c->world;
    t.slot_bytes = c->slot_bytes;
    t.seq = seq;
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

// slot of exchange `seq` of the current step (ctl[0] is stable for the whole step)
__device__ __forceinline__ int exchange_slot(const unsigned *ctl, int seq) {
  return (int)((ctl[0] + (unsigned)seq) % (unsigned)AR_SLOTS);
}
// byte offset of piece [rank] of this exchange's slot inside every receive buffer
__device__ __forceinline__ size_t push_piece_offset(const PushTarget &t) {
  return ((size_t)exchange_slot(t.ctl, t.seq) * t.world + t.rank) * t.slot_bytes;
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
