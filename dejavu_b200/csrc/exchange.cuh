// Tensor-parallel exchange: receiving side.
//
// Push protocol, the data is its own arrival flag. Every rank owns a receive buffer of AR_SLOTS slots x world
// pieces x slot_bytes, mapped into every peer with CUDA IPC and filled with a sentinel (fp16 -0.0, bits 0x8000).
//   * Sending: a rank stores its (B,d) fp16 partial sum into piece [rank] of the exchange's slot of EVERY rank
//     (plain stores over NVLink; -0.0 in the data is sent as +0.0, which changes no sum). The stores come from
//     the kernel that computed the partial (push.cuh) or from the consumer kernel itself.
//   * Receiving (this file): a block polls, bounded, the chunks it is responsible for in all pieces of the LOCAL
//     slot until no half of a chunk is the sentinel (a 16-byte store may arrive in parts, every half is
//     checked), adds the pieces in rank order in fp32 (same order on all ranks: bit-identical results
//     everywhere), rounds to fp16, adds the residual, and normalises.
//   * The blocks of a thread-block cluster split a row between them; the LayerNorm statistics are combined
//     through distributed shared memory (sum and centred second moment per block, merged exactly).
// One NVLink one-way trip per exchange, no fences, no remote loads, no flags.
// Numbering: exchange `seq` of a step uses slot (ctl[0] + seq) % AR_SLOTS; seq is fixed at launch (so a
// captured CUDA graph replays it) and ctl[0] is advanced once per step by djv_comm_end_step. See push.cuh for
// which kernel refills which slot and why that is safe.
// No multicast or multimem objects are used: a peer that exits between steps cannot fault the others, their
// next wait just runs out and reports DJV_ERR_TIMEOUT in the status word ctl[1].
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "push.cuh"

namespace djv {

namespace cg = cooperative_groups;

constexpr unsigned long long AR_WAIT_LIMIT_NS = 2000ull * 1000 * 1000;  // a wait on a peer gives up after 2 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct FoldArgs {
  void *const *bufs;   // device table of every rank's receive buffer
  unsigned *ctl;       // [0] exchanges of earlier steps, [1] status
  int rank, world;
  size_t slot_bytes;
  int seq;
  const __half *partial;   // this rank's (B,d) partial to send first, or null (a producer kernel sent it)
  const __half *residual;  // (B,d) or null
  __half *r_out;           // (B,d) or null: sum of the pieces + residual
  const __half *gamma, *beta;  // LayerNorm weights; gamma == null: no normalisation
  float eps;
  __half *y;               // (B,d) or null: normalised rows in global memory
  int refill;              // this kernel is the main-stream consumer: it refills slot + 2
  int B, d;
};

inline FoldArgs fold_args(const djv_comm *c, int seq) {
  FoldArgs f{};
  f.bufs = c->bufs_dev;
  f.ctl = c->ctl_dev;
  f.rank = c->rank;
  f.world = c->world;
  f.slot_bytes = c->slot_bytes;
  f.seq = seq;
  return f;
}

template <int THREADS>
__device__ __forceinline__ float block_sum_t(float v, float *red) {
  const int lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / WARP) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ void unpack8f(const uint4 &v, float (&f)[8]) {
  const float2 a = h2f(v.x), b = h2f(v.y), c = h2f(v.z), d = h2f(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
// round 8 fp32 values to fp16 (kept in f as the rounded values), returns the packed halves
__device__ __forceinline__ uint4 round8(float (&f)[8]) {
  __half2 o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) o[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = __half22float2(o[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
  return *reinterpret_cast<uint4 *>(o);
}

// What a fold needs from device memory before it can address its slot. ctl[0] only changes between steps (one
// tiny kernel after every stream of the step has been joined, many kernels before the first exchange of the next
// step), and the table of buffers never changes: both may be read BEFORE the wait on the predecessor kernel,
// which takes two dependent round trips to memory off the critical path. The status word is advisory.
struct FoldCtx {
  int slot;
  bool dead;
  char *local;
};
__device__ __forceinline__ FoldCtx fold_begin(const FoldArgs &a) {
  FoldCtx c;
  c.slot = exchange_slot(a.ctl, a.seq);
  c.dead = a.ctl[1] != 0u;  // once a wait has run out the exchange is dead: later calls do not wait again
  c.local = static_cast<char *>(a.bufs[a.rank]);
  return c;
}

// Per-thread state of a fold: the values of the thread's chunks and their LayerNorm weights.
template <int ITEMS>
struct FoldRegs {
  float vals[ITEMS][8];
  uint4 g[ITEMS], bt[ITEMS];
};

// Work split: this block owns 16-byte chunks [c_lo, c_hi) of rows [b_lo, b_lo + nb); item = it * THREADS + tid
// names (row b_lo + item / nseg, chunk c_lo + item % nseg).
#define DJV_FOLD_ITEM(it)                                 \
  const int item = (it) * THREADS + (int)threadIdx.x;     \
  const bool valid = item < nb * nseg;                    \
  const int row = b_lo + (valid ? item / nseg : 0);       \
  const int ch = c_lo + (valid ? item % nseg : 0);        \
  (void)row; (void)ch

// The LayerNorm weights are produced by no kernel: they may be fetched before the wait on the predecessor.
template <int THREADS, int ITEMS>
__device__ __forceinline__ void fold_fetch_affine(FoldRegs<ITEMS> &fr, const FoldArgs &a, int c_lo, int c_hi,
                                                  int b_lo, int nb) {
  const int nseg = c_hi - c_lo;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    DJV_FOLD_ITEM(it);
    if (valid && a.gamma != nullptr) {
      fr.g[it] = ld_cached16(a.gamma + (size_t)ch * 8);
      fr.bt[it] = ld_cached16(a.beta + (size_t)ch * 8);
    } else {
      fr.g[it] = make_uint4(0, 0, 0, 0);
      fr.bt[it] = make_uint4(0, 0, 0, 0);
    }
  }
}

// The receiving side of one exchange for this block's part of the rows, run by every block of a cluster whose
// blocks together cover all chunks of the rows [b_lo, b_lo + nb). Call it after griddepcontrol.wait.
//   writer   this cluster stores r_out / y to global memory (exactly one cluster per row should)
//   x_s      shared memory, [nb][nseg * 8] halves: the block's part of the normalised rows (or null)
//   refill_w / refill_n   this block is worker refill_w of refill_n of the slot refill (used when a.refill)
//   red: THREADS / 32 * nb * 3 floats, st: nb * 4 floats, stf: nb * 2 floats, failed_s: one int, all in shared
//   memory; ctx from fold_begin
// CLUSTERED = false: the block covers the whole rows by itself (csize 1, no cluster-wide barrier is executed).
// Contains cluster-wide barriers: every block of the cluster must call it, with the same nb.
// The caller must keep the block alive (a cluster barrier) until its peers have read st.
// Returns false when a wait ran out (the status word is set; outputs are then not written).
template <int THREADS, int ITEMS, bool CLUSTERED = true>
__device__ __forceinline__ bool exchange_fold(const FoldArgs &a, const FoldCtx &ctx, cg::cluster_group &cluster,
                                              int csize, int c_lo, int c_hi, int b_lo, int nb, bool writer,
                                              __half *x_s, int refill_w, int refill_n, FoldRegs<ITEMS> &fr,
                                              float *red, float *st, float *stf, int *failed_s) {
  const int tid = threadIdx.x;
  const int nseg = c_hi - c_lo;
  const int d = a.d;
  if (tid == 0) *failed_s = 0;
  const int slot = ctx.slot;
  const bool dead = ctx.dead;
  char *local = ctx.local;
  const size_t cur_off = (size_t)slot * a.world * a.slot_bytes;
  __syncthreads();

  // 1. send this rank's partial, unless the kernel that computed it has done so
  if (a.partial != nullptr && !dead) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      DJV_FOLD_ITEM(it);
      if (valid) {
        const size_t elem = (size_t)row * d + (size_t)ch * 8;
        uint4 v = *reinterpret_cast<const uint4 *>(a.partial + elem);
        v.x = no_sentinel2(v.x); v.y = no_sentinel2(v.y); v.z = no_sentinel2(v.z); v.w = no_sentinel2(v.w);
        const size_t off = cur_off + (size_t)a.rank * a.slot_bytes + elem * 2;
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p)
          if (p < a.world) st_sys16(static_cast<char *>(a.bufs[p]) + off, v);
      }
    }
  }
  // 2. the slot used two exchanges ago becomes free again: every piece, over the bytes its last exchange wrote
  //    (ctl[AR_CTL_EXTENT + slot], recorded by that exchange's refilling consumer, which ran earlier on this stream;
  //    the buffers start out all-sentinel, the records at 0). Not the whole slot: slots sized for a large batch
  //    would cost every single-row exchange megabytes of stores.
  if (a.refill && refill_n > 0 && !dead) {
    const int old_slot = (slot + 2) % AR_SLOTS;
    size_t ext = a.ctl[AR_CTL_EXTENT + old_slot];
    ext = ext < a.slot_bytes ? ext : a.slot_bytes;
    const size_t p16 = ext / 16, n16 = (size_t)a.world * p16;
    const size_t per = (n16 + refill_n - 1) / refill_n;
    const size_t lo = (size_t)refill_w * per, hi = (lo + per < n16) ? lo + per : n16;
    const uint4 s = make_uint4(AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2);
    char *old = local + (size_t)old_slot * a.world * a.slot_bytes;
    for (size_t c = lo + tid; c < hi; c += THREADS)
      *reinterpret_cast<uint4 *>(old + (c / p16) * a.slot_bytes + (c % p16) * 16) = s;
    if (refill_w == 0 && tid == 0) a.ctl[AR_CTL_EXTENT + slot] = (unsigned)((size_t)a.B * a.d * 2);
  }

  // 3. wait for the chunks of every piece, reduce in rank order, residual add. With few chunks per thread the
  //    loads of ALL of them are issued before any is looked at (one round trip instead of one per chunk).
  const unsigned long long t_start = global_timer_ns();
  bool gave_up = dead;
  constexpr bool BATCHED = ITEMS <= 2;
  uint4 vb[BATCHED ? ITEMS : 1][AR_MAX_WORLD];
  uint4 rb[BATCHED ? ITEMS : 1];
  if (BATCHED && !gave_up) {
#pragma unroll
    for (int it = 0; it < (BATCHED ? ITEMS : 1); ++it) {
      DJV_FOLD_ITEM(it);
      if (valid) {
        const size_t elem = (size_t)row * d + (size_t)ch * 8;
        rb[it] = a.residual ? *reinterpret_cast<const uint4 *>(a.residual + elem) : make_uint4(0, 0, 0, 0);
        const char *piece0 = local + cur_off + elem * 2;
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p)
          if (p < a.world) vb[it][p] = ld_sys16(piece0 + (size_t)p * a.slot_bytes);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    DJV_FOLD_ITEM(it);
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
    if (valid && !gave_up) {
      const size_t elem = (size_t)row * d + (size_t)ch * 8;
      const char *piece0 = local + cur_off + elem * 2;
      uint4 v[AR_MAX_WORLD];
      uint4 rres;
      unsigned missing = (1u << a.world) - 1u;
      if (BATCHED) {
        rres = rb[BATCHED ? it : 0];
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p) {
          if (p < a.world) {
            v[p] = vb[BATCHED ? it : 0][p];
            if (arrived16(v[p])) missing &= ~(1u << p);
          }
        }
      } else {
        // the residual chunk is requested before the wait on the peers, not after it
        rres = a.residual ? *reinterpret_cast<const uint4 *>(a.residual + elem) : make_uint4(0, 0, 0, 0);
      }
      // all missing pieces are requested together; only the ones not there yet are asked for again
      while (missing != 0u) {
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p)
          if (missing >> p & 1u) v[p] = ld_sys16(piece0 + (size_t)p * a.slot_bytes);
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p)
          if ((missing >> p & 1u) && arrived16(v[p])) missing &= ~(1u << p);
        if (missing != 0u && global_timer_ns() - t_start > AR_WAIT_LIMIT_NS) {
          gave_up = true;
          break;
        }
      }
      if (!gave_up) {
        float t[8];
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p) {  // rank order
          if (p < a.world) {
            unpack8f(v[p], t);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] += t[e];
          }
        }
        round8(f);  // the all-reduced activation is an fp16 tensor
        if (a.residual) {
          unpack8f(rres, t);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] += t[e];
        }
        const uint4 packed = round8(f);
        if (writer && a.r_out) *reinterpret_cast<uint4 *>(a.r_out + elem) = packed;
        if (a.gamma == nullptr) {  // no normalisation: the rows themselves are the result
          if (writer && a.y) *reinterpret_cast<uint4 *>(a.y + elem) = packed;
          if (x_s) *reinterpret_cast<uint4 *>(x_s + ((size_t)(row - b_lo) * nseg + (ch - c_lo)) * 8) = packed;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) fr.vals[it][e] = f[e];
  }
  if (gave_up) *failed_s = 1;
  __syncthreads();
  const bool failed = *failed_s != 0;
  if (failed && tid == 0 && !dead) atomicExch(&a.ctl[1], (unsigned)DJV_ERR_TIMEOUT);
  if (a.gamma == nullptr) return !failed;

  // 4. LayerNorm statistics: every warp takes the sum and the centred second moment of its own values (two
  //    passes over registers, shuffles only); the warps' and then the blocks' moments are merged exactly
  //    (groups g with n_g, sum_g, M2_g: M2 = sum_g M2_g + sum_g n_g (mean_g - mean)^2).
  //    red: [THREADS / 32][nb][3] floats.
  {
    const int lane = tid % WARP, warp = tid / WARP;
    for (int b = 0; b < nb; ++b) {
      float s = 0.f, cnt = 0.f;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        DJV_FOLD_ITEM(it);
        if (valid && row - b_lo == b) {
          cnt += 8.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) s += fr.vals[it][e];
        }
      }
      s = warp_sum(s);
      cnt = warp_sum(cnt);
      const float mean_w = cnt > 0.f ? s / cnt : 0.f;
      float q = 0.f;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        DJV_FOLD_ITEM(it);
        if (valid && row - b_lo == b) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float t = fr.vals[it][e] - mean_w;
            q += t * t;
          }
        }
      }
      q = warp_sum(q);
      if (lane == 0) {
        red[(warp * nb + b) * 3 + 0] = cnt;
        red[(warp * nb + b) * 3 + 1] = s;
        red[(warp * nb + b) * 3 + 2] = q;
      }
    }
    __syncthreads();
    // warps -> block: warp 0, lane w takes warp w's moments; all groups are merged at once
    // (M2 = sum of the groups' M2 + sum of n_g * (mean_g - mean)^2), so the order of the shuffles is the only
    // order there is, and it is the same in every block.
    if (tid < WARP) {
      for (int b = 0; b < nb; ++b) {
        float nw = 0.f, sw = 0.f, qw = 0.f;
        if (tid < THREADS / WARP) {
          nw = red[(tid * nb + b) * 3 + 0];
          sw = red[(tid * nb + b) * 3 + 1];
          qw = red[(tid * nb + b) * 3 + 2];
        }
        const float n = warp_sum(nw), sum = warp_sum(sw);
        const float mean = n > 0.f ? sum / n : 0.f;
        const float dm = nw > 0.f ? sw / nw - mean : 0.f;
        const float M2 = warp_sum(qw + nw * dm * dm);
        if (tid == 0) {
          st[b * 4 + 0] = sum;
          st[b * 4 + 1] = M2;
          st[b * 4 + 2] = n;
        }
      }
    }
  }
  if (CLUSTERED) cluster.sync(); else __syncthreads();
  // blocks -> row: lane j takes block j's moments (one round of remote reads), merged the same way
  if (tid < WARP) {
    for (int b = 0; b < nb; ++b) {
      float nj = 0.f, sj = 0.f, qj = 0.f;
      if (tid < csize) {
        const float *r = CLUSTERED ? cluster.map_shared_rank(st, tid) : st;
        sj = r[b * 4 + 0];
        qj = r[b * 4 + 1];
        nj = r[b * 4 + 2];
      }
      const float mean = warp_sum(sj) / (float)d;
      const float dm = nj > 0.f ? sj / nj - mean : 0.f;
      const float M2 = warp_sum(qj + nj * dm * dm);
      if (tid == 0) {
        stf[b * 2 + 0] = mean;
        stf[b * 2 + 1] = rsqrtf(M2 / (float)d + a.eps);
      }
    }
  }
  __syncthreads();
  if (failed) return false;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    DJV_FOLD_ITEM(it);
    if (valid) {
      const float mean = stf[(row - b_lo) * 2 + 0], rstd = stf[(row - b_lo) * 2 + 1];
      float gw[8], bw[8], o[8];
      unpack8f(fr.g[it], gw);
      unpack8f(fr.bt[it], bw);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (fr.vals[it][e] - mean) * rstd * gw[e] + bw[e];
      const uint4 packed = round8(o);
      if (writer && a.y) *reinterpret_cast<uint4 *>(a.y + (size_t)row * d + (size_t)ch * 8) = packed;
      if (x_s) *reinterpret_cast<uint4 *>(x_s + ((size_t)(row - b_lo) * nseg + (ch - c_lo)) * 8) = packed;
    }
  }
  return true;
}

}  // namespace djv
