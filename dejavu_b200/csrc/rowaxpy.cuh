// rowaxpy:  y[b,:] = sum_m x[b,m] * w[idx[m],:] + bias    (gather transposed GEMV, fc2 / out_proj shape)
//
// grid = (column tiles, 8*MCC), thread-block clusters of 8 along y.
//   * a block owns 256*CW consecutive columns (32 lanes x CW 16-byte chunks, 512 B apart) and its 8 warps own
//     disjoint slices of the index list: a warp streams its rows with 8 independent 128-bit loads in
//     flight per lane (8/CW rows x CW chunks) and keeps 8*CW*B fp32 sums per lane;
//   * the 8 warp sums are added through shared memory, the 8 blocks of a cluster through distributed
//     shared memory (plain ld.shared::cluster, each block finishing an eighth of the tile's columns);
//   * with MCC > 1 clusters per column tile the per-cluster sums go to `partial` and the last block to
//     arrive adds them in cluster order. Every sum has a fixed order: results are deterministic.
// Scratch: [4096 B of zeroed counters][MCC * B * N floats]. The kernel leaves the counters at zero.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "push.cuh"

namespace djv {

namespace cg = cooperative_groups;

constexpr int RA_THREADS = 256;
constexpr int RA_WARPS = RA_THREADS / WARP;
constexpr int RA_CLUSTER = 8;
constexpr int RA_MAX_MCC = 6;
constexpr int RA_COUNTER_BYTES = 4096;
constexpr int RA_MAX_B = 4;
constexpr int RA_MMA_MIN_B = 3;  // djv_gather_transposed_gemv: from this many rows of x on, the tensor-core kernel

// Last stage of rowaxpy_kernel:
// the block adds the 8 blocks' sums for its slice of columns and either stores them (one cluster per column
// tile) or leaves them in `partial` for the last block to arrive.
template <int B, int CW>
__device__ __forceinline__ void rowaxpy_finish_body(const float (*fin)[B][WARP * 8 * CW / RA_CLUSTER],
                                                    __half *__restrict__ Y, const __half *__restrict__ bias,
                                                    float *__restrict__ partial, unsigned *__restrict__ counters,
                                                    int N, int tile, int crank, int mcc, int MCC,
                                                    const PushTarget &push) {
  constexpr int RA_COLS = WARP * 8 * CW;
  constexpr int RA_SLICE = RA_COLS / RA_CLUSTER;
  __shared__ int is_last;
  const int tid = threadIdx.x;
  // a thread finishes 8 consecutive columns: one 16-byte store to Y, or to every rank's receive buffer
  const int gcol0 = tile * RA_COLS + crank * RA_SLICE;
  constexpr int G8 = RA_SLICE / 8;
  const int fb = tid / G8, fg = tid % G8;  // valid when tid < G8 * B
  const int gcol = gcol0 + fg * 8;         // N % 8 == 0: the 8 columns are all inside or all outside
  const bool finisher = tid < G8 * B && gcol < N;
  auto emit = [&](float (&v)[8]) {
    if (bias) {
      float t8[8];
      const uint4 bv = ld_cached16(bias + gcol);
      const float2 b0 = h2f(bv.x), b1 = h2f(bv.y), b2 = h2f(bv.z), b3 = h2f(bv.w);
      t8[0] = b0.x; t8[1] = b0.y; t8[2] = b1.x; t8[3] = b1.y; t8[4] = b2.x; t8[5] = b2.y; t8[6] = b3.x; t8[7] = b3.y;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += t8[e];
    }
    __half2 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
    const uint4 packed = *reinterpret_cast<uint4 *>(o);
    if (push.bufs != nullptr)
      push16(push, push_piece_offset(push), (size_t)fb * N + gcol, packed);
    else
      *reinterpret_cast<uint4 *>(Y + (size_t)fb * N + gcol) = packed;
  };
  // column-parallel sums (one thread per column), then 8 columns are packed per finishing thread
  __shared__ __align__(16) float outv[B][RA_SLICE];
  const int cb = tid / RA_SLICE, ccol = tid % RA_SLICE;  // valid when tid < RA_SLICE * B
  const bool summer = tid < RA_SLICE * B && gcol0 + ccol < N;
  if (summer) {
    float sum = 0.f;
#pragma unroll
    for (int src = 0; src < RA_CLUSTER; ++src) sum += fin[src][cb][ccol];
    if (MCC == 1)
      outv[cb][ccol] = sum;
    else
      __stcg(partial + ((size_t)mcc * B + cb) * N + gcol0 + ccol, sum);
  }
  if (MCC == 1) {
    __syncthreads();
    if (finisher) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = outv[fb][fg * 8 + e];
      emit(v);
    }
    return;
  }

  // several clusters per column tile: the last block to arrive for this slice of columns adds them
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
  if (summer) {
    float sum = 0.f;
    for (int c = 0; c < MCC; ++c) sum += __ldcg(partial + ((size_t)c * B + cb) * N + gcol0 + ccol);
    outv[cb][ccol] = sum;
  }
  __syncthreads();
  if (finisher) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = outv[fb][fg * 8 + e];
    emit(v);
  }
  if (tid == 0) counters[counter_id] = 0;  // ready for the next launch
}

// Out of line on purpose. Measured: with this stage inlined the compiler schedules the streaming loop of the
// kernel differently (fewer registers, fewer loads in flight) and fc2 runs 20-50 % slower, depending on B and on
// small details of this stage; behind a call the loop's code no longer depends on it.
template <int B, int CW>
__device__ __noinline__ void rowaxpy_finish_call(const float (*fin)[B][WARP * 8 * CW / RA_CLUSTER], __half *Y,
                                                 const __half *bias, float *partial, unsigned *counters, int N,
                                                 int tile, int crank, int mcc, int MCC, const PushTarget &push) {
  rowaxpy_finish_body<B, CW>(fin, Y, bias, partial, counters, N, tile, crank, mcc, MCC, push);
}

// CW: 16-byte chunks per lane along a row; a warp reads CW*512 contiguous bytes of every row it visits
template <int B, int CW>
__global__ void __cluster_dims__(1, RA_CLUSTER, 1) __launch_bounds__(RA_THREADS)
rowaxpy_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
               const void *__restrict__ idx, const __half *__restrict__ bias,
               float *__restrict__ partial, unsigned *__restrict__ counters, int M, int N,
               long long ldw, int idx64, int rows_per_warp, PushTarget push) {
  pdl_prologue();
  constexpr int RA_COLS = WARP * 8 * CW;           // columns per block
  constexpr int RA_SLICE = RA_COLS / RA_CLUSTER;   // columns a block finishes
  constexpr int U = 8 / CW;                        // rows in flight per lane: U * CW = 8 loads
  __shared__ __align__(16) float wsum[RA_WARPS][B][RA_COLS];
  __shared__ float tsum[B][RA_COLS];
  __shared__ float fin[RA_CLUSTER][B][RA_SLICE];

  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int tile = blockIdx.x;
  const int crank = blockIdx.y % RA_CLUSTER;  // rank inside the cluster
  const int mcc = blockIdx.y / RA_CLUSTER, MCC = gridDim.y / RA_CLUSTER;
  const int nchunks = N / 8;
  const int chunk0 = tile * WARP * CW + lane;  // this lane's chunks: chunk0 + c*32

  const int wslot = blockIdx.y * RA_WARPS + warp;
  const int m_begin = min(M, wslot * rows_per_warp);
  const int m_end = min(M, m_begin + rows_per_warp);

  float acc[B][CW][8];
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[b][c][e] = 0.f;

  const __half *wcol = W + (size_t)chunk0 * 8;
  for (int i0 = m_begin; i0 < m_end; i0 += WARP) {
    // lane l holds row i0+l of this warp's slice: its index and its x values
    // (fetching these further ahead of the weight stream was measured slower)
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
      uint4 wv[U][CW];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = __shfl_sync(0xffffffffu, my_row, (u0 + u) & 31);
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          if (chunk0 + c * WARP < nchunks && u0 + u < cnt)
            wv[u][c] = ld_stream16(wcol + (long long)r * ldw + c * WARP * 8);
          else
            wv[u][c] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int c = 0; c < CW; ++c) keep_loaded(wv[u][c]);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float xb[B];
        // rows past the end of the slice carry x = 0 and zero weights
#pragma unroll
        for (int b = 0; b < B; ++b) xb[b] = __shfl_sync(0xffffffffu, my_x[b], (u0 + u) & 31);
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          const float2 w0 = h2f(wv[u][c].x), w1 = h2f(wv[u][c].y), w2 = h2f(wv[u][c].z), w3 = h2f(wv[u][c].w);
#pragma unroll
          for (int b = 0; b < B; ++b) {
            acc[b][c][0] = fmaf(xb[b], w0.x, acc[b][c][0]);
            acc[b][c][1] = fmaf(xb[b], w0.y, acc[b][c][1]);
            acc[b][c][2] = fmaf(xb[b], w1.x, acc[b][c][2]);
            acc[b][c][3] = fmaf(xb[b], w1.y, acc[b][c][3]);
            acc[b][c][4] = fmaf(xb[b], w2.x, acc[b][c][4]);
            acc[b][c][5] = fmaf(xb[b], w2.y, acc[b][c][5]);
            acc[b][c][6] = fmaf(xb[b], w3.x, acc[b][c][6]);
            acc[b][c][7] = fmaf(xb[b], w3.y, acc[b][c][7]);
          }
        }
      }
    }
  }

  // 8 warps -> block
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int c = 0; c < CW; ++c) {
      float4 *dst = reinterpret_cast<float4 *>(&wsum[warp][b][(c * WARP + lane) * 8]);
      dst[0] = make_float4(acc[b][c][0], acc[b][c][1], acc[b][c][2], acc[b][c][3]);
      dst[1] = make_float4(acc[b][c][4], acc[b][c][5], acc[b][c][6], acc[b][c][7]);
    }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int c = 0; c < CW; ++c) {
      float s = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < RA_WARPS; ++w2) s += wsum[w2][b][c * RA_THREADS + tid];
      tsum[b][c * RA_THREADS + tid] = s;
    }
  // 8 blocks -> cluster: block `crank` finishes columns [crank*32, crank*32+32) of the tile
  cluster.sync();
#pragma unroll
  for (int c = 0; c < CW; ++c) {
    const int e = c * RA_THREADS + tid;
    const int src = e / RA_SLICE, col = e % RA_SLICE;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float *remote = cluster.map_shared_rank(&tsum[b][crank * RA_SLICE + col], src);
      fin[src][b][col] = *remote;
    }
  }
  cluster.sync();  // after this no block reads another block's shared memory any more

  rowaxpy_finish_call<B, CW>(fin, Y, bias, partial, counters, N, tile, crank, mcc, MCC, push);
}

struct RowaxpyPlan {
  int tiles, mcc, rpw, cw;
};

// Clusters of rowaxpy_kernel<B, CW> the device can hold at once (all GPCs together); 0 if the query fails.
template <int B, int CW>
inline int rowaxpy_query_clusters() {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, RA_CLUSTER, 1);
  cfg.blockDim = dim3(RA_THREADS, 1, 1);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = RA_CLUSTER;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, rowaxpy_kernel<B, CW>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// B in 1..4; cw as chosen by rowaxpy_chunks_per_lane(B). Cached: all devices of a process are the same model.
inline int rowaxpy_max_clusters(int B, int cw) {
  static int cache[RA_MAX_B + 1] = {0, 0, 0, 0, 0};
  if (B < 1 || B > RA_MAX_B) return 0;
  if (cache[B] == 0) {
    int n = 0;
    if (cw == 2) n = (B == 1) ? rowaxpy_query_clusters<1, 2>() : rowaxpy_query_clusters<2, 2>();
    else if (B == 1) n = rowaxpy_query_clusters<1, 1>();
    else if (B == 2) n = rowaxpy_query_clusters<2, 1>();
    else if (B == 3) n = rowaxpy_query_clusters<3, 1>();
    else n = rowaxpy_query_clusters<4, 1>();
    // fall-back: 2 blocks per multiprocessor, less what the cluster granularity of a GPC loses
    cache[B] = n > 0 ? n : (sm_count() * 2) / RA_CLUSTER * 7 / 8;
  }
  return cache[B];
}

// 16-byte chunks per lane: 1 KB contiguous per row and warp (measured faster than 512 B at equal grids)
// where the shared-memory reduction buffers still fit statically
inline int rowaxpy_chunks_per_lane(int B) {
  static const int k_cw = env_int("DJV_RA_CW", 2);  // development knob
  return (k_cw >= 2 && B <= 2) ? 2 : 1;
}

// One wave: as many clusters per column tile as the device holds at once. A grid that spills into a second,
// partly filled wave was measured 20-40% slower than a smaller grid that fits.
inline RowaxpyPlan plan_rowaxpy(int M, int N, int B) {
  const int cw = rowaxpy_chunks_per_lane(B);
  const int tiles = ceil_div(N / 8, WARP * cw);
  static const int k_mcc = env_int("DJV_RA_MCC", 0);  // development knob
  int mcc = k_mcc > 0 ? k_mcc : rowaxpy_max_clusters(B, cw) / tiles;
  if (mcc < 1) mcc = 1;
  if (mcc > RA_MAX_MCC) mcc = RA_MAX_MCC;
  // no point in splitting below ~8 rows per warp
  while (mcc > 1 && ceil_div(M, mcc * RA_CLUSTER * RA_WARPS) < 8) --mcc;
  const int rpw = ceil_div(M, mcc * RA_CLUSTER * RA_WARPS);
  return {tiles, mcc, rpw < 1 ? 1 : rpw, cw};
}

inline size_t rowaxpy_scratch_bytes(int B, int N, int M) {
  const RowaxpyPlan p = plan_rowaxpy(M, N, B);
  return RA_COUNTER_BYTES + (size_t)p.mcc * B * N * sizeof(float);
}

template <int B>
inline void launch_rowaxpy(const RowaxpyPlan &p, __half *Y, const __half *W, const __half *X,
                           const void *idx, const __half *bias, float *partial, unsigned *counters,
                           int M, int N, long long ldw, int idx64, cudaStream_t st, const PushTarget &push) {
  dim3 grid(p.tiles, p.mcc * RA_CLUSTER);
  if (p.cw == 2 && B <= 2)
    djv::launch_kernel(rowaxpy_kernel<(B <= 2 ? B : 1), 2>, grid, RA_THREADS, 0, st, Y, W, X, idx, bias, partial,
                       counters, M, N, ldw, idx64, p.rpw, push);
  else
    djv::launch_kernel(rowaxpy_kernel<B, 1>, grid, RA_THREADS, 0, st, Y, W, X, idx, bias, partial, counters, M, N,
                       ldw, idx64, p.rpw, push);
}

// B <= RA_MAX_B rows of x per launch
inline int rowaxpy_slice(int B, __half *Y, const __half *W, const __half *X, const void *idx,
                         const __half *bias, void *scratch, int M, int N, long long ldw, int idx64,
                         cudaStream_t st, const PushTarget &push = PushTarget{}) {
  const RowaxpyPlan p = plan_rowaxpy(M, N, B);
  if ((size_t)p.tiles * RA_CLUSTER * sizeof(unsigned) > RA_COUNTER_BYTES) {
    set_error("gather_transposed_gemv: N=%d needs more block counters than the scratch header holds", N);
    return DJV_ERR_UNSUPPORTED;
  }
  unsigned *counters = reinterpret_cast<unsigned *>(scratch);
  float *partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + RA_COUNTER_BYTES);
  switch (B) {
    case 1: launch_rowaxpy<1>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st, push); break;
    case 2: launch_rowaxpy<2>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st, push); break;
    case 3: launch_rowaxpy<3>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st, push); break;
    case 4: launch_rowaxpy<4>(p, Y, W, X, idx, bias, partial, counters, M, N, ldw, idx64, st, push); break;
    default: set_error("gather_transposed_gemv: internal batch slice %d", B); return DJV_ERR_INVALID;
  }
  return DJV_OK;
}

}  // namespace djv
