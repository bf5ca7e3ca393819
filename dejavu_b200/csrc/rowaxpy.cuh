// rowaxpy:  y[b,:] = sum_m x[b,m] * w[idx[m],:] + bias    (gather transposed GEMV, fc2 / out_proj shape)
//
// grid = (column tiles, 8*MCC), thread-block clusters of 8 along y.
//   * a block owns 256 consecutive columns (32 lanes x one 16-byte chunk) and its 8 warps own
//     disjoint slices of the index list: a warp streams its rows with 8 independent 128-bit loads in
//     flight per lane and keeps 8*B fp32 sums per lane;
//   * the 8 warp sums are added through shared memory, the 8 blocks of a cluster through distributed
//     shared memory (plain ld.shared::cluster, each block finishing 32 of the 256 columns);
//   * with MCC > 1 clusters per column tile the per-cluster sums go to `partial` and the last block to
//     arrive adds them in cluster order. Every sum has a fixed order: results are deterministic.
// Scratch: [4096 B of zeroed counters][MCC * B * N floats]. The kernel leaves the counters at zero.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace djv {

namespace cg = cooperative_groups;

constexpr int RA_THREADS = 256;
constexpr int RA_WARPS = RA_THREADS / WARP;
constexpr int RA_COLS = WARP * 8;  // columns per block
constexpr int RA_CLUSTER = 8;
constexpr int RA_SLICE = RA_COLS / RA_CLUSTER;  // columns a block finishes
constexpr int RA_MAX_MCC = 4;
constexpr int RA_COUNTER_BYTES = 4096;
constexpr int RA_MAX_B = 4;

template <int B>
__global__ void __cluster_dims__(1, RA_CLUSTER, 1) __launch_bounds__(RA_THREADS)
rowaxpy_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
               const void *__restrict__ idx, const __half *__restrict__ bias,
               float *__restrict__ partial, unsigned *__restrict__ counters, int M, int N,
               long long ldw, int idx64, int rows_per_warp) {
  pdl_prologue();
  __shared__ __align__(16) float wsum[RA_WARPS][B][RA_COLS];
  __shared__ float tsum[B][RA_COLS];
  __shared__ float fin[RA_CLUSTER][B][RA_SLICE];
  __shared__ int is_last;

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int tile = blockIdx.x;
  const int crank = blockIdx.y % RA_CLUSTER;  // rank inside the cluster
  const int mcc = blockIdx.y / RA_CLUSTER, MCC = gridDim.y / RA_CLUSTER;
  const int nchunks = N / 8;
  const int chunk = tile * WARP + lane;
  const bool active = chunk < nchunks;

  const int wslot = blockIdx.y * RA_WARPS + warp;
  const int m_begin = min(M, wslot * rows_per_warp);
  const int m_end = min(M, m_begin + rows_per_warp);

  float acc[B][8];
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[b][e] = 0.f;

  const __half *wcol = W + (size_t)chunk * 8;
  constexpr int U = 8;
  for (int i0 = m_begin; i0 < m_end; i0 += WARP) {
    // lane l holds row i0+l of this warp's slice: its index and its x values
    const int mi = i0 + lane;
    int my_row = 0;
    float my_x[B];
#pragma unroll
    for (int b = 0; b < B; ++b) my_x[b] = 0.f;
    if (mi < m_end) {
      my_row = (int)load_index(idx, mi, idx64);
#pragma unroll
      for (int b = 0; b < B; ++b) my_x[b] = __half2float(X[(size_t)b * M + mi]);
    }
    const int cnt = min(WARP, m_end - i0);
    for (int u0 = 0; u0 < cnt; u0 += U) {
      uint4 wv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = __shfl_sync(0xffffffffu, my_row, (u0 + u) & 31);
        if (active && u0 + u < cnt)
          wv[u] = ld_stream16(wcol + (long long)r * ldw);
        else
          wv[u] = make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float2 w0 = h2f(wv[u].x), w1 = h2f(wv[u].y), w2 = h2f(wv[u].z), w3 = h2f(wv[u].w);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          // rows past the end of the slice carry x = 0 and zero weights
          const float xb = __shfl_sync(0xffffffffu, my_x[b], (u0 + u) & 31);
          acc[b][0] = fmaf(xb, w0.x, acc[b][0]);
          acc[b][1] = fmaf(xb, w0.y, acc[b][1]);
          acc[b][2] = fmaf(xb, w1.x, acc[b][2]);
          acc[b][3] = fmaf(xb, w1.y, acc[b][3]);
          acc[b][4] = fmaf(xb, w2.x, acc[b][4]);
          acc[b][5] = fmaf(xb, w2.y, acc[b][5]);
          acc[b][6] = fmaf(xb, w3.x, acc[b][6]);
          acc[b][7] = fmaf(xb, w3.y, acc[b][7]);
        }
      }
    }
  }

  // 8 warps -> block
#pragma unroll
  for (int b = 0; b < B; ++b) {
    float4 *dst = reinterpret_cast<float4 *>(&wsum[warp][b][lane * 8]);
    dst[0] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
    dst[1] = make_float4(acc[b][4], acc[b][5], acc[b][6], acc[b][7]);
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < B; ++b) {
    float s = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < RA_WARPS; ++w2) s += wsum[w2][b][tid];
    tsum[b][tid] = s;
  }
  // 8 blocks -> cluster: block `crank` finishes columns [crank*32, crank*32+32) of the tile
  cluster.sync();
  {
    const int src = tid / RA_SLICE, col = tid % RA_SLICE;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float *remote = cluster.map_shared_rank(&tsum[b][crank * RA_SLICE + col], src);
      fin[src][b][col] = *remote;
    }
  }
  cluster.sync();  // after this no block reads another block's shared memory any more

  const int gcol0 = tile * RA_COLS + crank * RA_SLICE;
  if (tid < RA_SLICE * B) {
    const int b = tid / RA_SLICE, col = tid % RA_SLICE;
    float s = 0.f;
#pragma unroll
    for (int src = 0; src < RA_CLUSTER; ++src) s += fin[src][b][col];
    const int gcol = gcol0 + col;
    if (gcol < N) {
      if (MCC == 1) {
        Y[(size_t)b * N + gcol] = __float2half_rn(s + (bias ? __half2float(bias[gcol]) : 0.f));
      } else {
        __stcg(partial + ((size_t)mcc * B + b) * N + gcol, s);
      }
    }
  }
  if (MCC == 1) return;

  // several clusters per column tile: the last block to arrive for this 32-column slice adds them
  __threadfence();
  __syncthreads();
  const int counter_id = tile * RA_CLUSTER + crank;
  if (tid == 0) {
    const unsigned ticket = atomicAdd(&counters[counter_id], 1u);
    is_last = (ticket == (unsigned)MCC - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid < RA_SLICE * B) {
    const int b = tid / RA_SLICE, col = tid % RA_SLICE;
    const int gcol = gcol0 + col;
    if (gcol < N) {
      float s = 0.f;
      for (int c = 0; c < MCC; ++c) s += __ldcg(partial + ((size_t)c * B + b) * N + gcol);
      Y[(size_t)b * N + gcol] = __float2half_rn(s + (bias ? __half2float(bias[gcol]) : 0.f));
    }
  }
  if (tid == 0) counters[counter_id] = 0;  // ready for the next launch
}

struct RowaxpyPlan {
  int tiles, mcc, rpw;
};

inline RowaxpyPlan plan_rowaxpy(int M, int N) {
  const int sms = sm_count();
  const int tiles = ceil_div(N / 8, WARP);
  // aim at ~2.6 blocks of 256 threads per SM
  static const int k_blocks_x10 = env_int("DJV_RA_BLOCKS_X10", 26);  // development knob
  int mcc = (sms * k_blocks_x10 / 10 + tiles * RA_CLUSTER / 2) / (tiles * RA_CLUSTER);
  if (mcc < 1) mcc = 1;
  if (mcc > RA_MAX_MCC) mcc = RA_MAX_MCC;
  // no point in splitting below ~8 rows per warp
  while (mcc > 1 && ceil_div(M, mcc * RA_CLUSTER * RA_WARPS) < 8) --mcc;
  const int rpw = ceil_div(M, mcc * RA_CLUSTER * RA_WARPS);
  return {tiles, mcc, rpw < 1 ? 1 : rpw};
}

inline size_t rowaxpy_scratch_bytes(int B, int N, int M) {
  const RowaxpyPlan p = plan_rowaxpy(M, N);
  return RA_COUNTER_BYTES + (size_t)p.mcc * B * N * sizeof(float);
}

template <int B>
inline void launch_rowaxpy(const RowaxpyPlan &p, __half *Y, const __half *W, const __half *X,
                           const void *idx, const __half *bias, float *partial, unsigned *counters,
                           int M, int N, long long ldw, int idx64, cudaStream_t st) {
  dim3 grid(p.tiles, p.mcc * RA_CLUSTER);
  djv::launch_kernel(rowaxpy_kernel<B>, grid, RA_THREADS, 0, st, Y, W, X, idx, bias, partial, counters, M, N, ldw,
                                                 idx64, p.rpw);
}

// B <= RA_MAX_B rows of x per launch
inline int rowaxpy_slice(int B, __half *Y, const __half *W, const __half *X, const void *idx,
                         const __half *bias, void *scratch, int M, int N, long long ldw, int idx64,
                         cudaStream_t st) {
  const RowaxpyPlan p = plan_rowaxpy(M, N);
  if ((size_t)p.tiles * RA_CLUSTER * sizeof(unsigned) > RA_COUNTER_BYTES) {
    set_error("gather_transposed_gemv: N=%d needs more block counters than the scratch header holds", N);
    return DJV_ERR_UNSUPPORTED;
  }
  unsigned *counters = reinterpret_cast<unsigned *>(scratch);
  float *partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + RA_COUNTER_BYTES);
  switch (B) {
    case 1: launch_rowaxpy<1>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st); break;
    case 2: launch_rowaxpy<2>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st); break;
    case 3: launch_rowaxpy<3>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st); break;
    case 4: launch_rowaxpy<4>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st); break;
    default: set_error("gather_transposed_gemv: internal batch slice %d", B); return DJV_ERR_INVALID;
  }
  return DJV_OK;
}

}  // namespace djv
