// Device-resident state of the lazy K/V window of one attention layer, and the step that opens a decode
// step on it. Shared by the attention kernels and by the top-K kernel, which can run this step right after it
// has selected the heads (then no separate launch is needed on the critical path of the next layer).
#pragma once
#include "common.cuh"

namespace djv {

// state words, see DJV_ATTN_STATE_* in the header
enum { ST_SLOT = 0, ST_BASE = 1, ST_NEFF = 2, ST_STATUS = 3, ST_OPEN = 4 };  // ST_OPEN: a step awaits its advance
__device__ __forceinline__ int *st_pending(int *st) { return st + DJV_ATTN_STATE_HDR; }
__device__ __forceinline__ int *st_eff(int *st, int nheads) { return st + DJV_ATTN_STATE_HDR + nheads; }
__device__ __forceinline__ int *st_rowmask(int *st, int nheads) {
  return st + DJV_ATTN_STATE_HDR + 2 * nheads;
}

// Opens a decode step; call with a block of 1024 threads, all threads, once:
//   advance past the previous step if it was not closed, stash x in the window (when x != null), pick the heads
//   in use (head_idx[0..nnz), or ALL heads when head_idx == null or the window slot is the last one), emit
//   them in ascending order with the window slots each one has to compute, update `pending`.
__device__ __forceinline__ void attn_prep_block(int *__restrict__ st, const int *__restrict__ head_idx, int nnz,
                                                const __half *__restrict__ x, __half *__restrict__ x_ring, int d,
                                                int nheads, int S) {
  const int tid = threadIdx.x;
  int slot = st[ST_SLOT], base = st[ST_BASE];
  // the previous step was not closed by djv_attn_step_finish: advance past it first
  if (st[ST_OPEN] != 0 && st[ST_STATUS] == 0) {
    if (++slot >= DJV_KV_WINDOW) {
      slot = 0;
      base += DJV_KV_WINDOW;
    }
  }
  __syncthreads();  // every thread has read the old words
  if (tid == 0) {
    st[ST_SLOT] = slot;
    st[ST_BASE] = base;
    st[ST_OPEN] = 1;
  }
  int *pending = st_pending(st), *eff = st_eff(st, nheads), *rowmask = st_rowmask(st, nheads);
  const bool bad = slot < 0 || slot >= DJV_KV_WINDOW || base < 0 || base + slot >= S;
  if (bad) {
    if (tid == 0) {
      st[ST_STATUS] = DJV_ERR_INVALID;
      st[ST_NEFF] = 0;
    }
    return;
  }
  if (x != nullptr) {  // x_ring[slot] = x
    const uint4 *src = reinterpret_cast<const uint4 *>(x);
    uint4 *dst = reinterpret_cast<uint4 *>(x_ring + (size_t)slot * d);
    for (int c = tid; c < d / 8; c += blockDim.x) dst[c] = src[c];
  }

  const bool all = (head_idx == nullptr) || (slot == DJV_KV_WINDOW - 1);
  const int bit = 1 << slot;
  __shared__ int selected[1024];
  __shared__ int warp_tot[32];
  for (int h = tid; h < nheads; h += blockDim.x) selected[h] = all ? 1 : 0;
  __syncthreads();
  if (!all)
    for (int i = tid; i < nnz; i += blockDim.x) {
      const int h = head_idx[i];
      if (h >= 0 && h < nheads) selected[h] = 1;  // duplicates collapse here
    }
  __syncthreads();
  // heads in use are emitted in ascending head order: exclusive scan of the flags (nheads <= 1024)
  const int lane = tid % WARP, warp = tid / WARP;
  const int flag = (tid < nheads) ? selected[tid] : 0;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(ballot & ((1u << lane) - 1u));
  if (lane == 0) warp_tot[warp] = __popc(ballot);
  __syncthreads();
  int before = 0, total = 0;
  for (int w2 = 0; w2 < 32; ++w2) {
    const int t = warp_tot[w2];
    if (w2 < warp) before += t;
    total += t;
  }
  if (tid < nheads) {
    if (flag) {
      const int pos = before + in_warp;
      eff[pos] = tid;
      rowmask[pos] = pending[tid] | bit;
      pending[tid] = 0;
    } else {
      pending[tid] |= bit;
    }
  }
  if (tid == 0) st[ST_NEFF] = total;
}

}  // namespace djv
