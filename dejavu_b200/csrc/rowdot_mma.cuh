// rowdot_mma: gather GEMV for 9..32 rows of x on the tensor cores (mma.sync m16n8k16, fp16 in, fp32 accumulate).
//
//   y[b, m] = act( w[idx[m], :] . x[b, :] + bias[idx[m]] )
//
// With this many activation rows the gathered product is a real small-N contraction: per 16-byte weight
// chunk the CUDA-core kernel would issue 8*B FMAs, which no longer hides behind the HBM stream. Here a block
// owns 16 gathered rows; its 8 warps split the reduction dimension (warp w takes 32-element blocks w, w+8, ...),
// every lane loads 16 contiguous bytes of two of the rows and 16 bytes of one activation row per block, and two
// MMAs consume them. The 8 k-values a lane loads are not the ones the MMA fragment layout names, but weights and
// activations are permuted the same way along k, and a dot product does not care.
// Traffic is unchanged: every gathered row is read once.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace djv {

constexpr int MM_THREADS = 256;
constexpr int MM_WARPS = MM_THREADS / WARP;
constexpr int MM_ROWS = 16;

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Short index lists: M / 16 blocks would leave most of the device idle, so the reduction dimension is also split
// over the blocks of a thread-block cluster (grid (tiles, S), cluster (1, S), 1 <= S <= 8): block s of a cluster
// takes k-blocks s*8 + warp, then strides by 8*S; block 0 adds the others' sums through distributed shared memory, in block order.
// (Several 16-row tiles per block, to read the activations once for all of them, was measured 2-3 times slower at
// 16 and 32 activation rows: fewer, fatter blocks keep fewer loads in flight.)
// Blocks per multiprocessor the kernel is compiled for: a block's fixed costs (row numbers, first loads, the
// reduction at the end) overlap with other resident blocks' streaming, so more blocks of fewer registers per
// thread beat 4 blocks with deeper per-warp load pipelines (measured: K = 6144, 8 activation rows, 30 us against 42).
template <int NT>
struct MmaBlocks {
  static constexpr int PER_SM = NT == 1 ? 5 : 1;  // (1: whatever the compiler's register count allows, 4 here)
};

template <int NT, int ACT>  // NT groups of 8 activation rows
__global__ void __launch_bounds__(MM_THREADS, MmaBlocks<NT>::PER_SM)
rowdot_mma_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
                  const void *__restrict__ idx, const __half *__restrict__ bias, int M, int N,
                  long long ldw, int idx64, int B) {
  pdl_prologue();
  __shared__ float red[MM_WARPS][NT][MM_ROWS][8];
  __shared__ float bsum[NT][MM_ROWS][8];
  const int S = gridDim.y, sblk = blockIdx.y;
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int g = lane / 4, t = lane % 4;
  const int m0 = blockIdx.x * MM_ROWS;
  const int m_lo = m0 + g, m_hi = m0 + g + 8;
  const long long r_lo = (m_lo < M) ? load_index(idx, m_lo, idx64) : -1;
  const long long r_hi = (m_hi < M) ? load_index(idx, m_hi, idx64) : -1;
  const __half *w_lo = W + (r_lo < 0 ? 0 : r_lo) * ldw;
  const __half *w_hi = W + (r_hi < 0 ? 0 : r_hi) * ldw;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const int kblocks = (N + 31) / 32;
  // weight and activation loads of U k-blocks are all issued before the first MMA needs them
  constexpr int U = 2;
  for (int kb0 = sblk * MM_WARPS + warp; kb0 < kblocks; kb0 += MM_WARPS * S * U) {
    uint4 a_lo[U], a_hi[U], xv[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb0 + u * MM_WARPS * S) * 32 + t * 8;
      const bool ok = k < N;  // N % 8 == 0: a 16-byte piece is inside the row or entirely outside
      a_lo[u] = (ok && r_lo >= 0) ? ld_stream16(w_lo + k) : make_uint4(0, 0, 0, 0);
      a_hi[u] = (ok && r_hi >= 0) ? ld_stream16(w_hi + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int tok = j * 8 + g;
        xv[u][j] = (ok && tok < B) ? ld_cached16(X + (size_t)tok * N + k) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        // blocks past the end of the row hold zeros on both sides and add nothing
        mma_m16n8k16(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xv[u][j].x, xv[u][j].y);
        mma_m16n8k16(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xv[u][j].z, xv[u][j].w);
      }
    }
  }
  // acc[j]: rows g (e 0,1) and g+8 (e 2,3), tokens j*8 + 2t (e 0,2) and j*8 + 2t+1 (e 1,3)
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    red[warp][j][g][2 * t] = acc[j][0];
    red[warp][j][g][2 * t + 1] = acc[j][1];
    red[warp][j][g + 8][2 * t] = acc[j][2];
    red[warp][j][g + 8][2 * t + 1] = acc[j][3];
  }
  __syncthreads();
  namespace cgx = cooperative_groups;
  cgx::cluster_group cluster = cgx::this_cluster();
  if (S > 1) {
    // this block's sums, then the cluster's
    for (int o = tid; o < NT * MM_ROWS * 8; o += MM_THREADS) {
      const int j = o / (MM_ROWS * 8), row = (o / 8) % MM_ROWS, c = o % 8;
      float s = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < MM_WARPS; ++w2) s += red[w2][j][row][c];
      bsum[j][row][c] = s;
    }
    cluster.sync();
  }
  if (sblk == 0) {
    for (int o = tid; o < NT * MM_ROWS * 8; o += MM_THREADS) {
      const int j = o / (MM_ROWS * 8), row = (o / 8) % MM_ROWS, c = o % 8;
      const int m = m0 + row, tok = j * 8 + c;
      if (m < M && tok < B) {
        float s = 0.f;
        if (S > 1) {
          for (int q = 0; q < S; ++q) s += cluster.map_shared_rank(&bsum[0][0][0], q)[o];
        } else {
#pragma unroll
          for (int w2 = 0; w2 < MM_WARPS; ++w2) s += red[w2][j][row][c];
        }
        if (bias != nullptr) s += __half2float(bias[load_index(idx, m, idx64)]);
        Y[(size_t)tok * M + m] = __float2half_rn(apply_act<ACT>(s));
      }
    }
  }
  if (S > 1) cluster.sync();  // no block leaves while block 0 may still read its sums
}

template <int NT>
inline int launch_rowdot_mma(int act, __half *Y, const __half *W, const __half *X, const void *idx,
                             const __half *bias, int M, int N, long long ldw, int idx64, int B, cudaStream_t st) {
  const int tiles = ceil_div(M, MM_ROWS);
  // Split the reduction over the S blocks of a cluster when the tiles alone leave multiprocessors idle.
  static const int bps = [] {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, rowdot_mma_kernel<NT, DJV_ACT_RELU>, MM_THREADS, 0) !=
        cudaSuccess) {
      cudaGetLastError();
      n = 1;
    }
    return n < 1 ? 1 : n;
  }();
  const int slots = sm_count() * bps;
  // Measured behaviour: the resident blocks run in waves; a wave costs a fixed ~5 us (row numbers, first loads,
  // reduction, cluster barriers) plus, per k-block of 32 columns a warp walks, the larger of a latency floor that
  // grows with the activation rows and the wave's bytes per k-block step (8 KB per block) over the HBM rate.
  // S in {1, 2, 4, 8} (other cluster sizes measured slower than either neighbour), every warp keeps >= 4 k-blocks.
  const int kblocks = (N + 31) / 32;
  int S = 1;
  double best = 1e30;
  for (int c = 1; c <= 8; c *= 2) {
    if (c > 1 && kblocks < MM_WARPS * c * 4) break;
    const double kb_per_warp = (double)ceil_div(kblocks, MM_WARPS * c);
    const double floor_us = 0.6 + 0.23 * NT;
    double t = 0.0;
    for (int left = tiles * c; left > 0; left -= slots) {
      const int nb = left < slots ? left : slots;
      const double bw_us = nb * 8192.0 / 6.5e6;
      t += 5.0 + kb_per_warp * (floor_us > bw_us ? floor_us : bw_us);
    }
    if (t < best - 1e-9) {
      best = t;
      S = c;
    }
  }
  static const int k_s = env_int("DJV_MMA_S", 0);  // development knob
  if (k_s >= 1 && k_s <= 8) S = k_s;
  const dim3 grid(tiles, S), cluster(1, S, 1);
#define DJV_MM(ACT_)                                                                                              \
  djv::launch_kernel_cluster(rowdot_mma_kernel<NT, ACT_>, grid, dim3(MM_THREADS), 0, st, cluster, Y, W, X, idx, bias, \
                             M, N, ldw, idx64, B)
  switch (act) {
    case DJV_ACT_ID: DJV_MM(DJV_ACT_ID); break;
    case DJV_ACT_RELU: DJV_MM(DJV_ACT_RELU); break;
    case DJV_ACT_GELU: DJV_MM(DJV_ACT_GELU); break;
    case DJV_ACT_GELU_APPROX: DJV_MM(DJV_ACT_GELU_APPROX); break;
    case DJV_ACT_SQUARED_RELU: DJV_MM(DJV_ACT_SQUARED_RELU); break;
    default: set_error("gather_gemv: unknown activation %d", act); return DJV_ERR_INVALID;
  }
#undef DJV_MM
  return DJV_OK;
}

// 9 <= B <= 32
inline int rowdot_mma(int B, int act, __half *Y, const __half *W, const __half *X, const void *idx,
                      const __half *bias, int M, int N, long long ldw, int idx64, cudaStream_t st) {
  switch ((B + 7) / 8) {
    case 1: return launch_rowdot_mma<1>(act, Y, W, X, idx, bias, M, N, ldw, idx64, B, st);
    case 2: return launch_rowdot_mma<2>(act, Y, W, X, idx, bias, M, N, ldw, idx64, B, st);
    case 3: return launch_rowdot_mma<3>(act, Y, W, X, idx, bias, M, N, ldw, idx64, B, st);
    case 4: return launch_rowdot_mma<4>(act, Y, W, X, idx, bias, M, N, ldw, idx64, B, st);
  }
  set_error("gather_gemv: batch %d outside the tensor-core kernel's range", B);
  return DJV_ERR_INVALID;
}

}  // namespace djv
