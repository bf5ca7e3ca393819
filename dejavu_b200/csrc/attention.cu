// Head-sparse attention block for decode: QKV projection of selected heads (with lazy K/V back-fill),
// single-query attention over the fp16 caches for those heads, head-gathered output projection, and
// the device-resident lazy-K/V state machine.
//
// Cache layouts (one layer, as the reference keeps them for its decode kernel,
// Dejavu/src/ops/triton/attention_proj_sparse.py:540-546, 410-416):
//   K cache (B, nheads, hd/8, S, 8)   element (h, j, pos) at ((h*(hd/8) + j/8)*S + pos)*8 + j%8
//   V cache (B, nheads, S, hd)        element (h, pos, j) at (h*S + pos)*hd + j
//
// Algorithmic bytes: QKV 3*a*hd*d*2 (+bias, x); attention 2*a*len*hd*2; out_proj d*a*hd*2 (+bias, ctx, y).
#include <cooperative_groups.h>

#include "attn_state.cuh"
#include "common.cuh"
#include "push.cuh"
#include "rowdot_mma.cuh"

namespace djv {

namespace cg = cooperative_groups;

__global__ void attn_state_reset_kernel(int *st, int nheads, int prompt_len) {
  pdl_prologue();
  const int words = DJV_ATTN_STATE_WORDS(nheads);
  for (int i = threadIdx.x; i < words; i += blockDim.x) st[i] = 0;
  __syncthreads();
  if (threadIdx.x == 0) st[ST_BASE] = prompt_len;
}

// Step 1 of djv_attn_step as a kernel of its own (see attn_prep_block).
__global__ void __launch_bounds__(1024)
attn_prep_kernel(int *__restrict__ st, const int *__restrict__ head_idx, int nnz,
                 const __half *__restrict__ x, __half *__restrict__ x_ring, int d, int nheads, int S, int nseq,
                 long long seq_ring) {
  pdl_prologue();
  attn_prep_block(st, head_idx, nnz, x, x_ring, d, nheads, S);
  if (nseq > 1) {
    // the other sequences of the batch share this state; each has its own window: x_ring[b][slot] = x[b]
    __syncthreads();
    if (st[ST_STATUS] != 0) return;
    const int slot = st[ST_SLOT];
    const int per = d / 8;
    for (int c = threadIdx.x; c < (nseq - 1) * per; c += blockDim.x) {
      const int b = 1 + c / per, k = c % per;
      reinterpret_cast<uint4 *>(x_ring + (size_t)b * seq_ring + (size_t)slot * d)[k] =
          reinterpret_cast<const uint4 *>(x + (size_t)b * d)[k];
    }
  }
}

__global__ void attn_finish_kernel(int *st) {
  pdl_prologue();
  if (threadIdx.x == 0 && st[ST_STATUS] == 0 && st[ST_OPEN] != 0) {
    st[ST_OPEN] = 0;
    int slot = st[ST_SLOT] + 1;
    if (slot >= DJV_KV_WINDOW) {
      slot = 0;
      st[ST_BASE] += DJV_KV_WINDOW;
    }
    st[ST_SLOT] = slot;
  }
}

// ------------------------------------------------------------------------------------------
// QKV projection of selected heads for up to 16 token rows.
// A block owns QKV_RPB consecutive output rows j of one (head, q|k|v) pair, so every warp group in
// the block sees the same set of token rows and the block-wide barriers are uniform.
//   MODE 0: operator semantics (rows = batch_idx[i,:] >= 0, output y (T,3,nheads,hd))
//   MODE 1: decode step (rows = bits of rowmask[i]; q of the current slot -> q_out, K/V -> caches)
// ------------------------------------------------------------------------------------------
constexpr int QKV_THREADS = 256;
constexpr int QKV_WARPS = QKV_THREADS / WARP;

struct QkvArgs {
  const __half *w;     // (3,nheads,hd,d)
  const __half *bias;  // (3,nheads,hd) or null
  const __half *x;     // (T,d) or x_ring (16,d)
  int d, nheads, hd, nnz, T;
  // MODE 0
  __half *y;
  const int *head_idx;
  const int *batch_idx;
  // MODE 1
  int *state;
  __half *q_out, *k_cache, *v_cache;
  int S;
  // MODE 1 when the step was opened without the stash of x (djv_topk_attn_prep): the current token row is read
  // from x_cur, and block 0 copies it into the window for later back-fills. Null otherwise.
  const __half *x_cur;
  __half *x_ring_w;
  int early;  // MODE 1: the state is complete before this kernel can start; prefetch weights before the wait
  // MODE 1 with nseq sequences that share the state (same head selection, same window): elements between two
  // sequences' windows (x), query rows (q_out) and caches. Block (., y) takes sequences y*QKV_SEQ_GROUP ..: their
  // token rows go through the same pass over the weight rows, 16 at a time.
  int nseq;
  long long seq_x, seq_q, seq_k, seq_v;
};
constexpr int QKV_SEQ_GROUP = 8;  // sequences per block
// a token row of MODE 1: (sequence << 4) | window slot
__device__ __forceinline__ int row_seq(int code) { return code >> 4; }
__device__ __forceinline__ int row_slot(int code) { return code & (DJV_KV_WINDOW - 1); }
static_assert(DJV_KV_WINDOW == 16, "token-row codes keep the window slot in 4 bits");

// ROWS weight rows against NB token rows: every activation chunk is loaded (through L1) once and used for
// all ROWS weight rows, so L1 traffic per weight byte is NB / ROWS. Without that sharing a head with three
// pending token rows reads 3 bytes of x per byte of weight and the kernel is bound by L1 bandwidth, not HBM.
template <int NB, int WPR, int ROWS, int U>
__device__ __forceinline__ void multi_rowdot(const uint4 *const (&wp)[ROWS], const uint4 *const (&xp)[NB],
                                             int nchunks, int glane, float (&acc)[ROWS][NB]) {
  constexpr int GLANES = WARP * WPR;
#pragma unroll
  for (int j = 0; j < ROWS; ++j)
#pragma unroll
    for (int r = 0; r < NB; ++r) acc[j][r] = 0.f;
  for (int c0 = glane; c0 < nchunks; c0 += GLANES * U) {
    uint4 wv[ROWS][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * GLANES;
#pragma unroll
      for (int j = 0; j < ROWS; ++j) wv[j][u] = (c < nchunks) ? ld_stream16(wp[j] + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * GLANES;
      if (c < nchunks) {
#pragma unroll
        for (int r = 0; r < NB; ++r) {
          const uint4 xv = ld_cached16(xp[r] + c);
#pragma unroll
          for (int j = 0; j < ROWS; ++j) acc[j][r] = dot8(wv[j][u], xv, acc[j][r]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < ROWS; ++j)
#pragma unroll
    for (int r = 0; r < NB; ++r) acc[j][r] = warp_sum(acc[j][r]);
}

// Tensor-core path of one block's RPB weight rows against 1..16 token rows (current token + back-fill of K, V).
// With several token rows the CUDA-core path issues 8 FMAs per token row per 16-byte weight chunk and stops
// hiding behind the HBM stream; here the rows form m16n8k16 tiles: a tile is 16 weight rows (8 when RPB == 8,
// the upper half of the fragment stays zero), TILES tiles per block, the block's warps split the reduction
// dimension KW ways per tile. Lane (g, t) loads 16 contiguous bytes of weight rows g and g+8 and of token
// rows g and g+8; the k-permutation this implies is the same on both operands, so the dot products are unchanged.
// NT = 1: up to 8 token rows, NT = 2: up to 16.
template <int MODE, int RPB, int NT>
__device__ __forceinline__ void qkv_mma_rows(const QkvArgs &a, int qkv, int h, int jrow0, int nrows,
                                             const int *rows_s, int base, int cur_slot, float *red) {
  constexpr int TILES = (RPB == 32) ? 2 : 1;
  constexpr int KW = QKV_WARPS / TILES;
  constexpr bool HALF = (RPB == 8);
  constexpr int VALID = HALF ? 8 : 16;
  constexpr int U = (HALF && NT == 1) ? 8 : 4;  // weight loads in flight per lane: 8 (4 when HALF and NT == 2)
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int g = lane / 4, t = lane % 4;
  const int tile = warp / KW, kw = warp % KW;
  const size_t wrow = ((size_t)qkv * a.nheads + h) * a.hd + jrow0 + tile * 16 + g;
  const __half *w_lo = a.w + wrow * a.d;
  const __half *w_hi = w_lo + (size_t)8 * a.d;
  const __half *xr[NT];
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    xr[j] = nullptr;
    if (j * 8 + g < nrows) {
      const int code = rows_s[j * 8 + g];
      const int r = (MODE == 1) ? row_slot(code) : code;
      const __half *xs = (MODE == 1) ? a.x + (size_t)row_seq(code) * a.seq_x : a.x;
      xr[j] = (MODE == 1 && a.x_cur != nullptr && r == cur_slot) ? a.x_cur : xs + (size_t)r * a.d;
    }
  }

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const int kblocks = (a.d + 31) / 32;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int kb0 = kw; kb0 < kblocks; kb0 += KW * U) {
    uint4 a_lo[U], a_hi[U], bx[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb0 + u * KW) * 32 + t * 8;
      const bool ok = k < a.d;  // d % 8 == 0: a 16-byte piece is inside the row or entirely outside
      a_lo[u] = ok ? ld_stream16(w_lo + k) : zero;
      a_hi[u] = (ok && !HALF) ? ld_stream16(w_hi + k) : zero;
#pragma unroll
      for (int j = 0; j < NT; ++j) bx[u][j] = (ok && xr[j]) ? ld_cached16(xr[j] + k) : zero;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_m16n8k16(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, bx[u][j].x, bx[u][j].y);
        mma_m16n8k16(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, bx[u][j].z, bx[u][j].w);
      }
    }
  }
  // acc[j]: weight rows g (e 0,1) and g+8 (e 2,3), token rows j*8 + 2t (e 0,2) and j*8 + 2t+1 (e 1,3)
  // red[warp][j][row][token]
  float(*r4)[2][16][8] = reinterpret_cast<float(*)[2][16][8]>(red);
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    r4[warp][j][g][2 * t] = acc[j][0];
    r4[warp][j][g][2 * t + 1] = acc[j][1];
    r4[warp][j][g + 8][2 * t] = acc[j][2];
    r4[warp][j][g + 8][2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  for (int o = tid; o < TILES * NT * 16 * 8; o += QKV_THREADS) {
    const int c = o % 8, row = (o / 8) % 16, j = (o / 128) % NT, tl = o / (128 * NT);
    const int tok = j * 8 + c;
    if (row >= VALID || tok >= nrows) continue;
    float sum = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < KW; ++w2) sum += r4[tl * KW + w2][j][row][c];
    const int jj = jrow0 + tl * 16 + row;
    if (a.bias) sum += __half2float(a.bias[((size_t)qkv * a.nheads + h) * a.hd + jj]);
    const __half out = __float2half_rn(sum);
    const int code = rows_s[tok];
    const int trow = (MODE == 1) ? row_slot(code) : code;
    const size_t sq = (MODE == 1) ? (size_t)row_seq(code) : 0;
    if (MODE == 0) {
      a.y[(((size_t)trow * 3 + qkv) * a.nheads + h) * a.hd + jj] = out;
    } else if (qkv == 1) {
      const int pos = base + trow;
      a.k_cache[sq * a.seq_k + (((size_t)h * (a.hd / 8) + jj / 8) * a.S + pos) * 8 + jj % 8] = out;
    } else if (qkv == 2) {
      const int pos = base + trow;
      a.v_cache[sq * a.seq_v + ((size_t)h * a.S + pos) * a.hd + jj] = out;
    } else {
      a.q_out[sq * a.seq_q + (size_t)h * a.hd + jj] = out;
    }
  }
}

// A block owns RPB = (8 / WPR) * ROWS consecutive output rows j of one (head, q|k|v) pair: each group of WPR
// warps takes ROWS of them. Every group sees the same token rows, so the block-wide barriers are uniform.
template <int MODE, int WPR, int ROWS>
__global__ void __launch_bounds__(QKV_THREADS, 2) qkv_sparse_kernel(QkvArgs a) {
  constexpr int GROUPS = QKV_WARPS / WPR;
  constexpr int RPB = GROUPS * ROWS;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (MODE == 1 && RPB >= 8 && a.early) {
    // The step was opened by an earlier, completed kernel (the caller's promise): the head this block works on
    // is known, so the first 4 KB of each of its weight rows are requested while the LayerNorm before this
    // kernel is still running.
    const int jblocks_pf = a.hd / RPB;
    const int pair_pf = blockIdx.x / jblocks_pf, jb_pf = blockIdx.x % jblocks_pf;
    const int i_pf = pair_pf / 3, qkv_pf = pair_pf % 3;
    if (i_pf < a.state[ST_NEFF]) {
      const int h_pf = st_eff(a.state, a.nheads)[i_pf];
      const char *w0 = reinterpret_cast<const char *>(a.w + (((size_t)qkv_pf * a.nheads + h_pf) * a.hd + jb_pf * RPB) * a.d);
      const size_t row_bytes = (size_t)a.d * 2;
      constexpr int LINES = 32;  // 128-byte lines per row
      for (int l = threadIdx.x; l < RPB * LINES; l += QKV_THREADS) {
        const int row = l / LINES, line = l % LINES;
        if ((size_t)line * 128 < row_bytes) prefetch_l2(w0 + row * row_bytes + (size_t)line * 128);
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int U = (ROWS == 1) ? 8 : (ROWS == 2 ? 4 : 2);  // ROWS * U = 8 weight loads in flight per lane
  __shared__ float red[QKV_WARPS][ROWS][8];
  __shared__ int rows_s[QKV_SEQ_GROUP * DJV_KV_WINDOW];
  __shared__ int nrows_s;

  const int jblocks = a.hd / RPB;
  const int pair = blockIdx.x / jblocks;  // i*3 + qkv
  const int jb = blockIdx.x % jblocks;
  const int i = pair / 3, qkv = pair % 3;

  int n_eff, slot = 0, base = 0;
  if (MODE == 0) {
    n_eff = a.nnz;
  } else {
    n_eff = a.state[ST_NEFF];
    slot = a.state[ST_SLOT];
    base = a.state[ST_BASE];
    if (a.x_cur != nullptr && blockIdx.x == 0 && a.state[ST_STATUS] == 0) {
      // nobody reads window row `slot` in this kernel: the current token is taken from x_cur
      const uint4 *src = reinterpret_cast<const uint4 *>(a.x_cur);
      uint4 *dst = reinterpret_cast<uint4 *>(a.x_ring_w + (size_t)slot * a.d);
      for (int c = threadIdx.x; c < a.d / 8; c += QKV_THREADS) dst[c] = src[c];
    }
  }
  if (i >= n_eff) return;
  const int h = (MODE == 0) ? a.head_idx[i] : st_eff(a.state, a.nheads)[i];

  // the token rows this (head, q|k|v) pair computes
  if (threadIdx.x == 0) {
    int n = 0;
    if (MODE == 0) {
      for (int t = 0; t < a.T; ++t) {
        const int r = a.batch_idx[i * a.T + t];
        if (r >= 0) rows_s[n++] = r;
      }
    } else {
      // the sequences of this block, sequence-major (all of them have the same pending window slots)
      const int seq0 = blockIdx.y * QKV_SEQ_GROUP;
      const int seq1 = min(a.nseq > 0 ? a.nseq : 1, seq0 + QKV_SEQ_GROUP);
      const unsigned m = (qkv == 0) ? (1u << slot) : (unsigned)st_rowmask(a.state, a.nheads)[i];
      for (int sq = seq0; sq < seq1; ++sq)
        for (int s = 0; s <= slot; ++s)
          if (m >> s & 1u) rows_s[n++] = (sq << 4) | s;
    }
    nrows_s = n;
  }
  __syncthreads();
  const int nrows = nrows_s;
  if (nrows == 0) return;
  if constexpr (RPB >= 8) {
    // full or half tensor-core tiles; measured faster than the CUDA-core path below even for one token row
    __shared__ float red_mma[QKV_WARPS * 2 * 16 * 8];
    // 16 token rows per pass over the block's weight rows (one pass unless several sequences have rows pending)
    for (int r0 = 0; r0 < nrows; r0 += 16) {
      const int nr = min(16, nrows - r0);
      if (r0 > 0) __syncthreads();  // the reduction buffer of the pass before has been read
      if (nr <= 8) qkv_mma_rows<MODE, RPB, 1>(a, qkv, h, jb * RPB, nr, rows_s + r0, base, slot, red_mma);
      else qkv_mma_rows<MODE, RPB, 2>(a, qkv, h, jb * RPB, nr, rows_s + r0, base, slot, red_mma);
    }
    // (the CUDA-core path below is compiled for the one-row-per-block variant only)
  } else {

  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int group = warp / WPR, wig = warp % WPR, glane = wig * WARP + lane;
  const int nchunks = a.d / 8;
  const uint4 *Xv = reinterpret_cast<const uint4 *>(a.x);

  const int j0 = jb * RPB + group * ROWS;
  const size_t wrow0 = ((size_t)qkv * a.nheads + h) * a.hd + j0;
  const uint4 *wp[ROWS];
  float bv[ROWS];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) {
    wp[j] = reinterpret_cast<const uint4 *>(a.w + (wrow0 + j) * a.d);
    bv[j] = a.bias ? __half2float(a.bias[wrow0 + j]) : 0.f;
  }

  constexpr int NBMAX = 8;  // token rows per pass over the weights
  for (int r0 = 0; r0 < nrows; r0 += NBMAX) {
    const int nb = min(NBMAX, nrows - r0);
    float acc[ROWS][NBMAX];
    const uint4 *xp[NBMAX];
#pragma unroll
    for (int r = 0; r < NBMAX; ++r) {
      const int code = rows_s[r0 + (r < nb ? r : 0)];
      const int tr = (MODE == 1) ? row_slot(code) : code;
      const uint4 *xs = (MODE == 1) ? Xv + (size_t)row_seq(code) * (a.seq_x / 8) : Xv;
      xp[r] = (MODE == 1 && a.x_cur != nullptr && tr == slot) ? reinterpret_cast<const uint4 *>(a.x_cur)
                                                              : xs + (size_t)tr * nchunks;
    }
    if (nb == 1) {
      const uint4 *x1[1] = {xp[0]};
      float a1[ROWS][1];
      multi_rowdot<1, WPR, ROWS, U>(wp, x1, nchunks, glane, a1);
#pragma unroll
      for (int j = 0; j < ROWS; ++j) acc[j][0] = a1[j][0];
    } else if (nb == 2) {
      const uint4 *x2[2] = {xp[0], xp[1]};
      float a2[ROWS][2];
      multi_rowdot<2, WPR, ROWS, U>(wp, x2, nchunks, glane, a2);
#pragma unroll
      for (int j = 0; j < ROWS; ++j) {
        acc[j][0] = a2[j][0];
        acc[j][1] = a2[j][1];
      }
    } else if (nb <= 4) {
      const uint4 *x4[4] = {xp[0], xp[1], xp[2], xp[3]};
      float a4[ROWS][4];
      multi_rowdot<4, WPR, ROWS, U>(wp, x4, nchunks, glane, a4);
#pragma unroll
      for (int j = 0; j < ROWS; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[j][r] = a4[j][r];
    } else {
      multi_rowdot<NBMAX, WPR, ROWS, U>(wp, xp, nchunks, glane, acc);
    }
    if (WPR > 1) {
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
          for (int r = 0; r < NBMAX; ++r) red[warp][j][r] = acc[j][r];
      }
      // all groups run the same r0 trip counts, so this barrier is block-uniform
      __syncthreads();
      if (wig == 0 && lane == 0) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
          for (int r = 0; r < NBMAX; ++r) {
            float sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < WPR; ++w2) sum += red[group * WPR + w2][j][r];
            acc[j][r] = sum;
          }
      }
    }
    if (wig == 0 && lane == 0) {
#pragma unroll
      for (int jr = 0; jr < ROWS; ++jr) {
        const int j = j0 + jr;
        for (int r = 0; r < nb; ++r) {
          const __half out = __float2half_rn(acc[jr][r] + bv[jr]);
          const int code = rows_s[r0 + r];
          const int row = (MODE == 1) ? row_slot(code) : code;
          const size_t sq = (MODE == 1) ? (size_t)row_seq(code) : 0;
          if (MODE == 0) {
            a.y[(((size_t)row * 3 + qkv) * a.nheads + h) * a.hd + j] = out;
          } else if (qkv == 0) {
            a.q_out[sq * a.seq_q + (size_t)h * a.hd + j] = out;
          } else if (qkv == 1) {
            const int pos = base + row;
            a.k_cache[sq * a.seq_k + (((size_t)h * (a.hd / 8) + j / 8) * a.S + pos) * 8 + j % 8] = out;
          } else {
            const int pos = base + row;
            a.v_cache[sq * a.seq_v + ((size_t)h * a.S + pos) * a.hd + j] = out;
          }
        }
      }
    }
    if (WPR > 1) __syncthreads();
  }
  }  // RPB < 8
}

// ------------------------------------------------------------------------------------------
// Single-query attention for a list of heads, split over the cached tokens.
// grid = (head slots, batch, splits); 128 threads; the splits of one (head, batch) form a thread-block
// cluster. Each split leaves its partial (max, sum, out[hd]) in its own shared memory; after a cluster
// barrier split 0 reads them through distributed shared memory, combines and writes the fp16 context.
// No global scratch, no atomics.
// ------------------------------------------------------------------------------------------
constexpr int AT_THREADS = 128;
constexpr int AT_MAX_SPLITS = 8;          // portable cluster size
constexpr int AT_COUNTER_BYTES = 4096;

struct AttnArgs {
  __half *ctx;           // (B,nheads,hd)
  const __half *q;       // (B,nheads,hd)
  const __half *k_cache, *v_cache;
  const int *head_idx;   // explicit list or null (= identity)
  const int *state;      // when non-null: heads/n_eff/len come from the lazy-KV state
  int nnz, nheads, hd, S, len;
  float scale;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS) decode_attn_kernel(AttnArgs a) {
  pdl_prologue();
  constexpr int CH = HD / 8;           // 16-byte chunks per head row
  constexpr int RPI = AT_THREADS / CH; // V rows per iteration
  __shared__ float qs[HD];
  __shared__ float sc[AT_THREADS];
  __shared__ float redf[AT_THREADS / WARP];
  __shared__ float osum[RPI][HD];

  const int tid = threadIdx.x, lane = tid % WARP, warp = tid / WARP;
  const int i = blockIdx.x, b = blockIdx.y, sp = blockIdx.z, nsplit = gridDim.z;
  int n_eff = a.nnz, len = a.len;
  if (a.state) {
    n_eff = a.state[ST_NEFF];
    len = a.state[ST_BASE] + a.state[ST_SLOT] + 1;
  }
  if (i >= n_eff) return;
  int h;
  if (a.state)
    h = a.state[DJV_ATTN_STATE_HDR + a.nheads + i];
  else
    h = a.head_idx ? a.head_idx[i] : i;

  const size_t bh = (size_t)b * a.nheads + h;
  const __half *Kh = a.k_cache + bh * (size_t)a.S * HD;
  const __half *Vh = a.v_cache + bh * (size_t)a.S * HD;

  const int chunk = (len + nsplit - 1) / nsplit;
  const int t_begin = min(len, sp * chunk), t_end = min(len, t_begin + chunk);

  float m_run = -INFINITY, l_run = 0.f;
  float oacc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) oacc[e] = 0.f;
  const int vrow = tid / CH, vch = tid % CH;
  const uint4 zero = make_uint4(0, 0, 0, 0);

  // A pass covers AT_THREADS tokens: thread t scores token t (CH 16-byte loads of K) and, for P.V, thread
  // (vrow, vch) reads chunk vch of V rows vrow, vrow+RPI, ... (CH loads). All 2*CH loads of a pass, and q in the
  // first pass, are issued before anything waits on them, so a pass costs one trip to HBM instead of three.
  for (int p0 = t_begin; p0 < t_end; p0 += AT_THREADS) {
    const int pn = min(AT_THREADS, t_end - p0);
    uint4 kreg[CH], vreg[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c)
      kreg[c] = (tid < pn) ? ld_stream16(Kh + ((size_t)c * a.S + p0 + tid) * 8) : zero;
#pragma unroll
    for (int it = 0; it < CH; ++it) {
      const int t = it * RPI + vrow;
      vreg[it] = (t < pn) ? ld_stream16(Vh + (size_t)(p0 + t) * HD + vch * 8) : zero;
    }
    if (p0 == t_begin) {
      for (int j = tid; j < HD; j += AT_THREADS) qs[j] = __half2float(a.q[bh * HD + j]) * a.scale;
      __syncthreads();
    }
    float s = -INFINITY;
    if (tid < pn) {
      s = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const float2 k0 = h2f(kreg[c].x), k1 = h2f(kreg[c].y), k2 = h2f(kreg[c].z), k3 = h2f(kreg[c].w);
        s = fmaf(qs[c * 8 + 0], k0.x, s);
        s = fmaf(qs[c * 8 + 1], k0.y, s);
        s = fmaf(qs[c * 8 + 2], k1.x, s);
        s = fmaf(qs[c * 8 + 3], k1.y, s);
        s = fmaf(qs[c * 8 + 4], k2.x, s);
        s = fmaf(qs[c * 8 + 5], k2.y, s);
        s = fmaf(qs[c * 8 + 6], k3.x, s);
        s = fmaf(qs[c * 8 + 7], k3.y, s);
      }
    }
    float lmax = warp_max(s);
    if (lane == 0) redf[warp] = lmax;
    __syncthreads();
    float m_new = m_run;
#pragma unroll
    for (int w2 = 0; w2 < AT_THREADS / WARP; ++w2) m_new = fmaxf(m_new, redf[w2]);
    __syncthreads();
    const float p = (tid < pn) ? __expf(s - m_new) : 0.f;
    sc[tid] = p;
    float lsum = warp_sum(p);
    if (lane == 0) redf[warp] = lsum;
    __syncthreads();  // sc[] and redf[] complete
    float ltot = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < AT_THREADS / WARP; ++w2) ltot += redf[w2];
    const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
    l_run = l_run * corr + ltot;
#pragma unroll
    for (int e = 0; e < 8; ++e) oacc[e] *= corr;
    m_run = m_new;
#pragma unroll
    for (int it = 0; it < CH; ++it) {
      const float pw = sc[it * RPI + vrow];  // 0 for tokens past the end of the pass
      const float2 v0 = h2f(vreg[it].x), v1 = h2f(vreg[it].y), v2 = h2f(vreg[it].z), v3 = h2f(vreg[it].w);
      oacc[0] = fmaf(pw, v0.x, oacc[0]);
      oacc[1] = fmaf(pw, v0.y, oacc[1]);
      oacc[2] = fmaf(pw, v1.x, oacc[2]);
      oacc[3] = fmaf(pw, v1.y, oacc[3]);
      oacc[4] = fmaf(pw, v2.x, oacc[4]);
      oacc[5] = fmaf(pw, v2.y, oacc[5]);
      oacc[6] = fmaf(pw, v3.x, oacc[6]);
      oacc[7] = fmaf(pw, v3.y, oacc[7]);
    }
    __syncthreads();  // sc[] and redf[] are reused by the next pass
  }
  // reduce the RPI row groups
#pragma unroll
  for (int e = 0; e < 8; ++e) osum[vrow][vch * 8 + e] = oacc[e];
  __syncthreads();
  float o = 0.f;  // thread j < HD owns output dim j
  if (tid < HD) {
#pragma unroll
    for (int r = 0; r < RPI; ++r) o += osum[r][tid];
  }

  if (nsplit == 1) {
    if (tid < HD) a.ctx[bh * HD + tid] = __float2half_rn(l_run > 0.f ? o / l_run : 0.f);
    return;
  }
  // the cluster spans the whole z extent of the grid: block rank in the cluster == sp.
  // Every block of a cluster took the same branch at `i >= n_eff`, so the barriers are cluster-uniform.
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float part_s[HD + 2];
  if (tid < HD) part_s[2 + tid] = o;
  if (tid == 0) {
    part_s[0] = m_run;
    part_s[1] = l_run;
  }
  cluster.sync();
  if (sp == 0 && tid < HD) {
    float ms[AT_MAX_SPLITS];
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) {
      ms[s] = (s < nsplit) ? *cluster.map_shared_rank(&part_s[0], s) : -INFINITY;
      m = fmaxf(m, ms[s]);
    }
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) {
      if (s < nsplit && ms[s] != -INFINITY) {
        const float w = __expf(ms[s] - m);
        l += w * *cluster.map_shared_rank(&part_s[1], s);
        acc += w * *cluster.map_shared_rank(&part_s[2 + tid], s);
      }
    }
    a.ctx[bh * HD + tid] = __float2half_rn(l > 0.f ? acc / l : 0.f);
  }
  cluster.sync();  // no block leaves while split 0 may still read its shared memory
}

// ------------------------------------------------------------------------------------------
// Output projection over selected heads, weight in the reference's (d, nheads, hd) layout: every output
// row n reads one contiguous hd*2-byte segment per selected head. A warp owns OP_ROWS output rows;
// hd/8 lanes cover one segment, so 32/(hd/8) segments are fetched per warp instruction.
// ------------------------------------------------------------------------------------------
constexpr int OP_THREADS = 256;
constexpr int OP_ROWS = 4;

template <int HD, int B>
__global__ void __launch_bounds__(OP_THREADS)
out_proj_sparse_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
                       const int *__restrict__ head_idx, const int *__restrict__ n_active_dev,
                       const __half *__restrict__ bias, int d, int nheads, int nnz, PushTarget push,
                       int early) {
  constexpr int LPS = HD / 8;      // lanes per segment
  constexpr int SEGS = WARP / LPS; // segments per warp load
  const int tid = threadIdx.x, lane = tid % WARP;
  const int gw = (blockIdx.x * OP_THREADS + tid) / WARP;
  const int n0 = gw * OP_ROWS;
  const int seg = lane / LPS, c = lane % LPS;
  const size_t row_stride = (size_t)nheads * HD;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (early && n0 < d) {
    // The head list is complete (the caller's promise): while the attention kernel before this one is still
    // running, ask for every weight segment this warp is going to read. One lane per 128-byte line.
    int n_pf = nnz;
    if (n_active_dev) n_pf = min(nnz, *n_active_dev);
    if (c % 8 == 0) {
      for (int i = seg; i < n_pf; i += SEGS) {
        const int h = head_idx[i];
#pragma unroll
        for (int r = 0; r < OP_ROWS; ++r)
          if (n0 + r < d) prefetch_l2(W + (size_t)(n0 + r) * row_stride + (size_t)h * HD + c * 8);
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (n0 >= d) return;
  int n_eff = nnz;
  if (n_active_dev) n_eff = min(nnz, *n_active_dev);

  float acc[OP_ROWS][B];
#pragma unroll
  for (int r = 0; r < OP_ROWS; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) acc[r][b] = 0.f;

  // two head segments per lane and iteration: 2 * OP_ROWS independent 16-byte loads in flight
  for (int i0 = seg; i0 < n_eff; i0 += SEGS * 2) {
    int h[2];
    bool ok[2];
    uint4 wv[2][OP_ROWS];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = i0 + k * SEGS;
      ok[k] = i < n_eff;
      h[k] = ok[k] ? head_idx[i] : 0;
#pragma unroll
      for (int r = 0; r < OP_ROWS; ++r) {
        const int n = n0 + r;
        wv[k][r] = (ok[k] && n < d) ? ld_stream16(W + (size_t)n * row_stride + (size_t)h[k] * HD + c * 8)
                                    : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (ok[k]) {
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const uint4 xv = ld_cached16(X + ((size_t)b * nheads + h[k]) * HD + c * 8);
#pragma unroll
          for (int r = 0; r < OP_ROWS; ++r) acc[r][b] = dot8(wv[k][r], xv, acc[r][b]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < OP_ROWS; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) acc[r][b] = warp_sum(acc[r][b]);
  if (lane == 0) {
    if (push.bufs != nullptr) {
      // this rank's partial goes straight into every rank's receive buffer, 4 rows (8 bytes) at a time;
      // d % 4 == 0, so the warp's 4 rows are all inside or all outside
      static_assert(OP_ROWS == 4, "the push path packs 4 rows into one 8-byte store");
      const size_t piece = push_piece_offset(push);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float v[OP_ROWS];
#pragma unroll
        for (int r = 0; r < OP_ROWS; ++r) v[r] = acc[r][b] + (bias ? __half2float(bias[n0 + r]) : 0.f);
        __half2 o[2] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3])};
        push8(push, piece, (size_t)b * d + n0, *reinterpret_cast<uint2 *>(o));
      }
    } else {
#pragma unroll
      for (int r = 0; r < OP_ROWS; ++r) {
        const int n = n0 + r;
        if (n < d) {
          const float bv = bias ? __half2float(bias[n]) : 0.f;
#pragma unroll
          for (int b = 0; b < B; ++b) Y[(size_t)b * d + n] = __float2half_rn(acc[r][b] + bv);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// cache scatter operators (reference semantics)
// ------------------------------------------------------------------------------------------
template <bool IS_K>
__global__ void cache_copy_sparse_kernel(const __half *__restrict__ src, __half *__restrict__ cache,
                                         const int *__restrict__ head_idx,
                                         const int *__restrict__ seqlen_idx,
                                         const int *__restrict__ padding, int T, int nheads, int hd,
                                         int S, long long ld_t, long long ld_h) {
  pdl_prologue();
  const int i = blockIdx.x, t = blockIdx.y;
  const int pos0 = seqlen_idx[i * T + t];
  if (pos0 < 0) return;
  const int h = head_idx[i];
  const int pos = pos0 + (padding ? *padding : 0);
  if (pos < 0 || pos >= S) return;
  // the source row is the token row named by seqlen_idx (the reference indexes k with it too)
  const __half *s = src + (size_t)pos0 * ld_t + (size_t)h * ld_h;
  for (int j = threadIdx.x; j < hd; j += blockDim.x) {
    if (IS_K)
      cache[(((size_t)h * (hd / 8) + j / 8) * S + pos) * 8 + j % 8] = s[j];
    else
      cache[((size_t)h * S + pos) * hd + j] = s[j];
  }
}

}  // namespace djv

using namespace djv;

// `rows` = output rows expected in a typical call (heads in use x 3 x head_dim). Blocks of 32, 16 or 8 weight
// rows run on the tensor cores with the block's 8 warps splitting the reduction dimension; the block size is
// the largest that still gives every multiprocessor about two blocks. Very small calls put a whole block on
// one row.
template <int MODE>
static void launch_qkv(QkvArgs a, int capacity_heads, long long rows, cudaStream_t st, int nseq = 1) {
  const long long sms = sm_count();
  // development knob, read at every launch: DJV_QKV_RPB (32, 16, 8 or 1: force the rows-per-block variant)
  const int force = env_int("DJV_QKV_RPB", 0);
  int rpb = (rows >= 32 * sms) ? 32 : (rows >= 16 * sms) ? 16 : (rows >= 2 * sms) ? 8 : 1;
  if (force == 32 || force == 16 || force == 8 || force == 1) rpb = force;
  if (a.hd % rpb != 0) rpb = 8;
#define DJV_QKV(WPR_, ROWS_)                                                                       \
  djv::launch_kernel(qkv_sparse_kernel<MODE, WPR_, ROWS_>,                                         \
                     dim3(capacity_heads * 3 * (a.hd / ((QKV_WARPS / WPR_) * ROWS_)), (nseq + QKV_SEQ_GROUP - 1) / QKV_SEQ_GROUP), \
                     QKV_THREADS, 0, st, a)
  if (rpb == 32) DJV_QKV(1, 4);
  else if (rpb == 16) DJV_QKV(2, 4);
  else if (rpb == 8) DJV_QKV(2, 2);
  else DJV_QKV(8, 1);
#undef DJV_QKV
}

static int check_hd(const char *op, int hd, int d) {
  DJV_REQUIRE(hd == 32 || hd == 64 || hd == 128, "%s: head_dim %d not in {32,64,128}", op, hd);
  DJV_REQUIRE(d >= 8 && d % 8 == 0, "%s: hidden dim %d must be a multiple of 8", op, d);
  return DJV_OK;
}

extern "C" int djv_qkv_proj_sparse(void *y, const void *w, const void *x, const int32_t *head_idx,
                                   const int32_t *batch_idx, const void *bias, int T, int d,
                                   int nheads, int hd, int nnz, void *stream) {
  DJV_REQUIRE(y && w && x && head_idx && batch_idx, "qkv_proj_sparse: null pointer");
  int rc = check_hd("qkv_proj_sparse", hd, d);
  if (rc) return rc;
  DJV_REQUIRE(T >= 1 && T <= DJV_KV_WINDOW, "qkv_proj_sparse: %d token rows outside [1,16]", T);
  DJV_REQUIRE(nnz >= 0 && nnz <= nheads, "qkv_proj_sparse: nnz=%d outside [0,%d]", nnz, nheads);
  DJV_REQUIRE(aligned16(w) && aligned16(x), "qkv_proj_sparse: w and x must be 16-byte aligned");
  if (nnz == 0) return DJV_OK;
  QkvArgs a{};
  a.w = static_cast<const __half *>(w);
  a.bias = static_cast<const __half *>(bias);
  a.x = static_cast<const __half *>(x);
  a.d = d; a.nheads = nheads; a.hd = hd; a.nnz = nnz; a.T = T;
  a.y = static_cast<__half *>(y);
  a.head_idx = head_idx;
  a.batch_idx = batch_idx;
  launch_qkv<0>(a, nnz, (long long)nnz * 3 * hd, static_cast<cudaStream_t>(stream));
  count_launch();
  return check_launch("qkv_proj_sparse");
}

template <int HD>
static int launch_out_proj(int B, __half *Y, const __half *W, const __half *X, const int *head_idx,
                           const int *n_active_dev, const __half *bias, int d, int nheads, int nnz,
                           cudaStream_t st, const PushTarget &push = PushTarget{}) {
  const int early = early_prefetch() ? 1 : 0;
  const int warps = ceil_div(d, OP_ROWS);
  const int grid = ceil_div(warps * WARP, OP_THREADS);
#define DJV_OP(B_) \
  djv::launch_kernel(out_proj_sparse_kernel<HD, B_>, grid, OP_THREADS, 0, st, Y, W, X, head_idx, n_active_dev, bias, d, nheads, nnz, push, early)
  switch (B) {
    case 1: DJV_OP(1); break;
    case 2: DJV_OP(2); break;
    case 3: DJV_OP(3); break;
    case 4: DJV_OP(4); break;
    case 8: DJV_OP(8); break;
    default: set_error("out_proj_sparse: internal batch slice %d", B); return DJV_ERR_INVALID;
  }
#undef DJV_OP
  return DJV_OK;
}

extern "C" int djv_out_proj_sparse(void *y, const void *w, const void *x, const int32_t *head_idx,
                                   const int32_t *n_active_dev, const void *bias, int B, int d,
                                   int nheads, int hd, int nnz, void *stream) {
  DJV_REQUIRE(y && w && x && (head_idx || nnz == 0), "out_proj_sparse: null pointer");
  int rc = check_hd("out_proj_sparse", hd, d);
  if (rc) return rc;
  DJV_REQUIRE(B >= 1 && B <= 16, "out_proj_sparse: batch %d outside [1,16]", B);
  DJV_REQUIRE(nnz >= 0 && nnz <= nheads, "out_proj_sparse: nnz=%d outside [0,%d]", nnz, nheads);
  DJV_REQUIRE(aligned16(w) && aligned16(x), "out_proj_sparse: w and x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // slices of 8 rows of x while 8 are left, then of up to 4 (each slice reads the selected columns once)
  for (int b0 = 0, bs = 0; b0 < B; b0 += bs) {
    bs = (B - b0 >= 8) ? 8 : ((B - b0 < 4) ? (B - b0) : 4);
    __half *Y = static_cast<__half *>(y) + (size_t)b0 * d;
    const __half *X = static_cast<const __half *>(x) + (size_t)b0 * nheads * hd;
    const __half *W = static_cast<const __half *>(w);
    const __half *bi = static_cast<const __half *>(bias);
    if (hd == 128) rc = launch_out_proj<128>(bs, Y, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st);
    else if (hd == 64) rc = launch_out_proj<64>(bs, Y, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st);
    else rc = launch_out_proj<32>(bs, Y, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st);
    if (rc) return rc;
    count_launch();
  }
  return check_launch("out_proj_sparse");
}

// The same projection with the result sent into every rank's receive buffer of the tensor-parallel exchange
// instead of y, as exchange number `seq` of the step (see push.cuh): the NVLink trip overlaps the kernel's
// tail, and the consumer of that exchange is called with partial == NULL.
extern "C" int djv_out_proj_sparse_push(djv_comm *comm, int seq, const void *w, const void *x, const int32_t *head_idx,
                                        const int32_t *n_active_dev, const void *bias, int B, int d,
                                        int nheads, int hd, int nnz, void *stream) {
  DJV_REQUIRE(comm && w && x && (head_idx || nnz == 0), "out_proj_sparse_push: null pointer");
  DJV_REQUIRE(seq >= 0, "out_proj_sparse_push: negative exchange number %d", seq);
  int rc = check_hd("out_proj_sparse_push", hd, d);
  if (rc) return rc;
  DJV_REQUIRE(B >= 1 && B <= 4, "out_proj_sparse_push: batch %d outside [1,4]", B);
  DJV_REQUIRE((size_t)B * d * 2 <= comm->slot_bytes, "out_proj_sparse_push: %zu bytes exceed the slot (%zu)",
              (size_t)B * d * 2, comm->slot_bytes);
  DJV_REQUIRE(nnz >= 0 && nnz <= nheads, "out_proj_sparse_push: nnz=%d outside [0,%d]", nnz, nheads);
  DJV_REQUIRE(aligned16(w) && aligned16(x), "out_proj_sparse_push: w and x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half *W = static_cast<const __half *>(w), *X = static_cast<const __half *>(x);
  const __half *bi = static_cast<const __half *>(bias);
  const PushTarget push = push_target(comm, seq);
  if (hd == 128) rc = launch_out_proj<128>(B, nullptr, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st, push);
  else if (hd == 64) rc = launch_out_proj<64>(B, nullptr, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st, push);
  else rc = launch_out_proj<32>(B, nullptr, W, X, head_idx, n_active_dev, bi, d, nheads, nnz, st, push);
  if (rc) return rc;
  count_launch();
  return check_launch("out_proj_sparse_push");
}

static int cache_copy(bool is_k, const void *src, void *cache, const int32_t *head_idx,
                      const int32_t *seqlen_idx, const int32_t *padding, int T, int nheads, int hd,
                      int S, int nnz, long long ld_t, long long ld_h, void *stream) {
  const char *op = is_k ? "k_cache_copy_sparse" : "v_cache_copy_sparse";
  DJV_REQUIRE(src && cache && head_idx && seqlen_idx, "%s: null pointer", op);
  DJV_REQUIRE(hd % 8 == 0 && hd >= 8, "%s: head_dim %d must be a multiple of 8", op, hd);
  DJV_REQUIRE(T >= 1 && T <= DJV_KV_WINDOW, "%s: %d token rows outside [1,16]", op, T);
  DJV_REQUIRE(nnz >= 0 && nnz <= nheads && S >= 1, "%s: bad nnz/S", op);
  if (nnz == 0) return DJV_OK;
  dim3 grid(nnz, T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_k)
    djv::launch_kernel(cache_copy_sparse_kernel<true>, grid, 128, 0, st, static_cast<const __half *>(src),
                                                         static_cast<__half *>(cache), head_idx,
                                                         seqlen_idx, padding, T, nheads, hd, S, ld_t, ld_h);
  else
    djv::launch_kernel(cache_copy_sparse_kernel<false>, grid, 128, 0, st, static_cast<const __half *>(src),
                                                          static_cast<__half *>(cache), head_idx,
                                                          seqlen_idx, padding, T, nheads, hd, S, ld_t, ld_h);
  count_launch();
  return check_launch(op);
}

extern "C" int djv_k_cache_copy_sparse(const void *k, void *k_cache, const int32_t *head_idx,
                                       const int32_t *seqlen_idx, const int32_t *padding, int T,
                                       int nheads, int hd, int S, int nnz, long long ld_t,
                                       long long ld_h, void *stream) {
  return cache_copy(true, k, k_cache, head_idx, seqlen_idx, padding, T, nheads, hd, S, nnz, ld_t, ld_h, stream);
}
extern "C" int djv_v_cache_copy_sparse(const void *v, void *v_cache, const int32_t *head_idx,
                                       const int32_t *seqlen_idx, const int32_t *padding, int T,
                                       int nheads, int hd, int S, int nnz, long long ld_t,
                                       long long ld_h, void *stream) {
  return cache_copy(false, v, v_cache, head_idx, seqlen_idx, padding, T, nheads, hd, S, nnz, ld_t, ld_h, stream);
}

extern "C" int djv_attn_state_reset(int32_t *state, int nheads, int prompt_len, void *stream) {
  DJV_REQUIRE(state && nheads >= 1 && nheads <= 1024 && prompt_len >= 0, "attn_state_reset: bad argument");
  djv::launch_kernel(attn_state_reset_kernel, 1, 256, 0, static_cast<cudaStream_t>(stream), state, nheads, prompt_len);
  count_launch();
  return check_launch("attn_state_reset");
}

static int attn_splits(int S) {
  int s = ceil_div(S, 128);
  if (s > AT_MAX_SPLITS) s = AT_MAX_SPLITS;
  if (s < 1) s = 1;
  return s;
}

static size_t attn_scratch_bytes(int slots, int B, int hd, int S) {
  return AT_COUNTER_BYTES + (size_t)slots * B * attn_splits(S) * (hd + 2) * sizeof(float);
}

// `scratch` is not used any more (the splits combine through distributed shared memory); the parameters stay
// in the C signatures so that existing callers keep working.
static int launch_attn(AttnArgs a, int slots, int B, void *scratch, size_t scratch_bytes, cudaStream_t st,
                       const char *op) {
  (void)scratch; (void)scratch_bytes; (void)op;
  const int nsplit = attn_splits(a.S);
  dim3 grid(slots, B, nsplit), cluster(1, 1, nsplit);
  if (a.hd == 128) djv::launch_kernel_cluster(decode_attn_kernel<128>, grid, AT_THREADS, 0, st, cluster, a);
  else if (a.hd == 64) djv::launch_kernel_cluster(decode_attn_kernel<64>, grid, AT_THREADS, 0, st, cluster, a);
  else djv::launch_kernel_cluster(decode_attn_kernel<32>, grid, AT_THREADS, 0, st, cluster, a);
  count_launch();
  return DJV_OK;
}

extern "C" size_t djv_attn_step_scratch_bytes(int nheads, int hd, int S) {
  if (nheads < 1 || hd < 8 || S < 1) return 0;
  return attn_scratch_bytes(nheads, 1, hd, S);
}

// B sequences in lockstep that share `state` (one head selection, one window position): q_out (B,nheads,hd),
// x (B,d), x_ring (B,16,d), caches (B,...) contiguous over the batch.
static int attn_step_project(void *q_out, const void *wqkv, const void *bqkv, const void *x, void *x_ring,
                             void *k_cache, void *v_cache, int32_t *state, const int32_t *head_idx, int nnz, int d,
                             int nheads, int hd, int S, int B, int step_is_open, void *stream) {
  DJV_REQUIRE(q_out && wqkv && x && x_ring && k_cache && v_cache && state, "attn_step: null pointer");
  int rc = check_hd("attn_step", hd, d);
  if (rc) return rc;
  DJV_REQUIRE(B >= 1 && B <= 65535, "attn_step: batch %d outside [1,65535]", B);
  DJV_REQUIRE(nheads >= 1 && nheads <= 1024, "attn_step: nheads=%d outside [1,1024]", nheads);
  DJV_REQUIRE(head_idx == nullptr || (nnz >= 0 && nnz <= nheads), "attn_step: nnz=%d outside [0,%d]", nnz, nheads);
  DJV_REQUIRE(S >= 1, "attn_step: cache capacity S=%d", S);
  DJV_REQUIRE(aligned16(wqkv) && aligned16(x) && aligned16(x_ring) && aligned16(k_cache) && aligned16(v_cache),
              "attn_step: pointers must be 16-byte aligned");
  DJV_REQUIRE(B == 1 || !step_is_open, "attn_step: a batch opens its step itself");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long seq_ring = (long long)DJV_KV_WINDOW * d;
  if (!step_is_open) {
    djv::launch_kernel(attn_prep_kernel, 1, 1024, 0, st, state, head_idx, head_idx ? nnz : 0,
                       static_cast<const __half *>(x), static_cast<__half *>(x_ring), d, nheads, S, B, seq_ring);
    count_launch();
  }
  QkvArgs a{};
  a.w = static_cast<const __half *>(wqkv);
  a.bias = static_cast<const __half *>(bqkv);
  a.x = static_cast<const __half *>(x_ring);
  a.d = d; a.nheads = nheads; a.hd = hd; a.nnz = nheads; a.T = DJV_KV_WINDOW;
  a.state = state;
  a.q_out = static_cast<__half *>(q_out);
  a.k_cache = static_cast<__half *>(k_cache);
  a.v_cache = static_cast<__half *>(v_cache);
  a.S = S;
  a.nseq = B;
  a.seq_x = seq_ring;
  a.seq_q = (long long)nheads * hd;
  a.seq_k = (long long)nheads * hd * S;
  a.seq_v = (long long)nheads * hd * S;
  if (step_is_open) {
    a.x_cur = static_cast<const __half *>(x);
    a.x_ring_w = static_cast<__half *>(x_ring);
    a.early = early_prefetch() ? 1 : 0;
  }
  const int typical = head_idx ? (nnz > 0 ? nnz : 1) : nheads;
  launch_qkv<1>(a, nheads, (long long)typical * 3 * hd, st, B);
  count_launch();
  return check_launch("attn_step_project");
}

extern "C" int djv_attn_step_project(void *q_out, const void *wqkv, const void *bqkv, const void *x,
                                     void *x_ring, void *k_cache, void *v_cache, int32_t *state,
                                     const int32_t *head_idx, int nnz, int d, int nheads, int hd, int S,
                                     int step_is_open, void *stream) {
  return attn_step_project(q_out, wqkv, bqkv, x, x_ring, k_cache, v_cache, state, head_idx, nnz, d, nheads, hd, S, 1,
                           step_is_open, stream);
}

extern "C" int djv_attn_step_project_batch(void *q_out, const void *wqkv, const void *bqkv, const void *x,
                                           void *x_ring, void *k_cache, void *v_cache, int32_t *state,
                                           const int32_t *head_idx, int nnz, int d, int nheads, int hd, int S,
                                           int B, void *stream) {
  return attn_step_project(q_out, wqkv, bqkv, x, x_ring, k_cache, v_cache, state, head_idx, nnz, d, nheads, hd, S, B,
                           0, stream);
}

static int attn_step_attend(void *ctx, const void *q, const void *k_cache, const void *v_cache, int32_t *state,
                            int B, int nheads, int hd, int S, float softmax_scale, void *scratch,
                            size_t scratch_bytes, void *stream) {
  DJV_REQUIRE(ctx && q && k_cache && v_cache && state, "attn_step: null pointer");
  DJV_REQUIRE(hd == 32 || hd == 64 || hd == 128, "attn_step: head_dim %d not in {32,64,128}", hd);
  DJV_REQUIRE(B >= 1 && B <= 65535, "attn_step: batch %d outside [1,65535]", B);
  DJV_REQUIRE(nheads >= 1 && nheads <= 1024, "attn_step: nheads=%d outside [1,1024]", nheads);
  DJV_REQUIRE(S >= 1, "attn_step: cache capacity S=%d", S);
  DJV_REQUIRE(aligned16(k_cache) && aligned16(v_cache), "attn_step: pointers must be 16-byte aligned");
  AttnArgs t{};
  t.ctx = static_cast<__half *>(ctx);
  t.q = static_cast<const __half *>(q);
  t.k_cache = static_cast<const __half *>(k_cache);
  t.v_cache = static_cast<const __half *>(v_cache);
  t.state = state;
  t.nnz = nheads; t.nheads = nheads; t.hd = hd; t.S = S; t.len = 0;
  t.scale = softmax_scale;
  int rc = launch_attn(t, nheads, B, scratch, scratch_bytes, static_cast<cudaStream_t>(stream), "attn_step");
  if (rc) return rc;
  return check_launch("attn_step_attend");
}

extern "C" int djv_attn_step_attend(void *ctx, const void *q, const void *k_cache, const void *v_cache,
                                    int32_t *state, int nheads, int hd, int S, float softmax_scale,
                                    void *scratch, size_t scratch_bytes, void *stream) {
  return attn_step_attend(ctx, q, k_cache, v_cache, state, 1, nheads, hd, S, softmax_scale, scratch, scratch_bytes,
                          stream);
}

extern "C" int djv_attn_step_attend_batch(void *ctx, const void *q, const void *k_cache, const void *v_cache,
                                          int32_t *state, int B, int nheads, int hd, int S, float softmax_scale,
                                          void *scratch, size_t scratch_bytes, void *stream) {
  return attn_step_attend(ctx, q, k_cache, v_cache, state, B, nheads, hd, S, softmax_scale, scratch, scratch_bytes,
                          stream);
}

extern "C" int djv_attn_step(void *ctx, void *q_out, const void *wqkv, const void *bqkv, const void *x,
                             void *x_ring, void *k_cache, void *v_cache, int32_t *state,
                             const int32_t *head_idx, int nnz, int d, int nheads, int hd, int S,
                             float softmax_scale, void *scratch, size_t scratch_bytes, void *stream) {
  DJV_REQUIRE(ctx != nullptr, "attn_step: null pointer");
  int rc = djv_attn_step_project(q_out, wqkv, bqkv, x, x_ring, k_cache, v_cache, state, head_idx, nnz, d, nheads,
                                 hd, S, 0, stream);
  if (rc) return rc;
  return djv_attn_step_attend(ctx, q_out, k_cache, v_cache, state, nheads, hd, S, softmax_scale, scratch,
                              scratch_bytes, stream);
}

extern "C" int djv_attn_step_finish(int32_t *state, int nheads, void *stream) {
  DJV_REQUIRE(state && nheads >= 1, "attn_step_finish: bad argument");
  djv::launch_kernel(attn_finish_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), state);
  count_launch();
  return check_launch("attn_step_finish");
}

extern "C" size_t djv_decode_attn_scratch_bytes(int nnz, int B, int hd, int S) {
  if (nnz < 1 || B < 1 || hd < 8 || S < 1) return 0;
  return attn_scratch_bytes(nnz, B, hd, S);
}

extern "C" int djv_decode_attn(void *ctx, const void *q, const void *k_cache, const void *v_cache,
                               const int32_t *head_idx, int nnz, int B, int nheads, int hd, int S,
                               int len, float softmax_scale, void *scratch, size_t scratch_bytes,
                               void *stream) {
  DJV_REQUIRE(ctx && q && k_cache && v_cache, "decode_attn: null pointer");
  DJV_REQUIRE(hd == 32 || hd == 64 || hd == 128, "decode_attn: head_dim %d not in {32,64,128}", hd);
  DJV_REQUIRE(B >= 1 && nheads >= 1 && S >= 1 && len >= 0 && len <= S, "decode_attn: bad sizes");
  const int slots = head_idx ? nnz : nheads;
  DJV_REQUIRE(slots >= 0 && slots <= nheads, "decode_attn: nnz=%d outside [0,%d]", nnz, nheads);
  DJV_REQUIRE(aligned16(k_cache) && aligned16(v_cache), "decode_attn: caches must be 16-byte aligned");
  if (slots == 0) return DJV_OK;
  AttnArgs t{};
  t.ctx = static_cast<__half *>(ctx);
  t.q = static_cast<const __half *>(q);
  t.k_cache = static_cast<const __half *>(k_cache);
  t.v_cache = static_cast<const __half *>(v_cache);
  t.head_idx = head_idx;
  t.nnz = slots; t.nheads = nheads; t.hd = hd; t.S = S; t.len = len;
  t.scale = softmax_scale;
  int rc = launch_attn(t, slots, B, scratch, scratch_bytes, static_cast<cudaStream_t>(stream), "decode_attn");
  if (rc) return rc;
  return check_launch("decode_attn");
}
