// Gather GEMV kernels for the sparse MLP (and, with idx == NULL, every dense GEMV of the decode step).
//
// Both kernels are bound by HBM bandwidth: each gathered weight row is read exactly once with 128-bit
// loads that bypass L1, accumulated in fp32 and rounded to fp16 once.
//
//   rowdot  : y[b,m] = act(w[idx[m],:] . x[b,:] + bias[idx[m]])      one row -> one output  (fc1)
//   rowaxpy : y[b,:] = sum_m x[b,m] * w[idx[m],:] + bias             one row -> a d-vector  (fc2)
//
// Algorithmic bytes per launch (fp16, int32 idx):
//   rowdot  : M*N*2 + M*2 (bias) + M*4 (idx) + B*N*2 (x) + B*M*2 (y)
//   rowaxpy : M*N*2 + B*M*2 (x) + N*2 (bias) + B*N*2 (y)
#include "common.cuh"
#include "rowaxpy.cuh"
#include "rowdot_mma.cuh"
#include "rowaxpy_mma.cuh"

namespace djv {

// the same products on the bulk-copy ring pipeline (mlp_ring.cu)
int ring_fc1(__half *y, const __half *w, const __half *x, const void *idx, const __half *bias, int B, int N, int M,
             long long ldw, int idx64, int act, cudaStream_t st);
int ring_fc2(__half *y, const __half *w, const __half *h, const void *idx, const __half *bias, int B, int N, int M,
             long long ldw, int idx64, void *scratch, cudaStream_t st, const PushTarget &push);
// Development knob DJV_RING_GEMV (read at every call): route djv_gather_gemv / djv_gather_transposed_gemv calls
// of at most that many rows through the ring pipeline when the shape allows it. 0 = never.
static int ring_gemv_rows() { return env_int("DJV_RING_GEMV", 0); }
static bool ring_shape_ok(int B, int N, int M) { return djv_mlp_sparse_fused_supported(B, N, M) != 0; }

// -------------------------------------------------------------------------------------------
// rowdot. A block has 8 warps split into 8/WPR groups of WPR warps; a group owns ROWS rows at a
// time and its 32*WPR lanes stride over the 16-byte chunks of those rows, U chunks in flight per
// lane per row. x is read through L1 (it is tiny and reused by every warp); weights bypass L1.
// Small M uses large WPR so that the whole device has loads in flight for a handful of rows.
// -------------------------------------------------------------------------------------------
constexpr int RD_THREADS = 256;
constexpr int RD_WARPS = RD_THREADS / WARP;

template <int B, int ACT, int WPR, int ROWS, int U>
__global__ void __launch_bounds__(RD_THREADS)
rowdot_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
              const void *__restrict__ idx, const __half *__restrict__ bias, int M, int N,
              long long ldw, int idx64, int early) {
  constexpr int GROUPS = RD_WARPS / WPR;
  constexpr int GLANES = WARP * WPR;
  __shared__ float red[WPR > 1 ? RD_WARPS * ROWS * B : 1];

  const int tid = threadIdx.x;
  const int warp = tid / WARP, lane = tid % WARP;
  const int group = warp / WPR, wig = warp % WPR;
  const int glane = wig * WARP + lane;
  const int nchunks = N / 8;
  const uint4 *Xv = reinterpret_cast<const uint4 *>(X);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (early) {
    // Weights are not produced by any kernel, and the index list is complete (identity, or the caller's
    // promise): the first 8 KB of the first rows of this group are requested while the kernel before this
    // one is still running.
    const int m0 = blockIdx.x * GROUPS * ROWS + group * ROWS;
    constexpr int LINES = 64;
    const int row_lines = (int)min((long long)LINES, ((long long)N * 2 + 127) / 128);
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      if (m0 + j < M) {
        const long long r = load_index(idx, m0 + j, idx64);
        const char *w0 = reinterpret_cast<const char *>(W + r * ldw);
        for (int l = glane; l < row_lines; l += GLANES) prefetch_l2(w0 + (size_t)l * 128);
      }
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int rows_per_pass = gridDim.x * GROUPS * ROWS;
  // trip count is uniform over the block so that __syncthreads below is legal
  for (int base = blockIdx.x * GROUPS * ROWS; base < M; base += rows_per_pass) {
    const int m0 = base + group * ROWS;
    const uint4 *wp[ROWS];
    float bv[ROWS];
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const int m = m0 + j;
      const bool ok = m < M;
      const long long r = ok ? load_index(idx, m, idx64) : 0;
      wp[j] = reinterpret_cast<const uint4 *>(W + r * ldw);
      bv[j] = (bias != nullptr && ok) ? __half2float(bias[r]) : 0.f;
      if (!ok) wp[j] = nullptr;
    }
    float acc[ROWS][B];
#pragma unroll
    for (int j = 0; j < ROWS; ++j)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[j][b] = 0.f;

    for (int c0 = glane; c0 < nchunks; c0 += GLANES * U) {
      uint4 wv[ROWS][U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * GLANES;
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
          if (c < nchunks && wp[j] != nullptr)
            wv[j][u] = ld_stream16(wp[j] + c);
          else
            wv[j][u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * GLANES;
        if (c < nchunks) {
#pragma unroll
          for (int b = 0; b < B; ++b) {
            const uint4 xv = ld_cached16(Xv + (size_t)b * nchunks + c);
#pragma unroll
            for (int j = 0; j < ROWS; ++j) acc[j][b] = dot8(wv[j][u], xv, acc[j][b]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < ROWS; ++j)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[j][b] = warp_sum(acc[j][b]);

    if (WPR > 1) {
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
          for (int b = 0; b < B; ++b) red[(warp * ROWS + j) * B + b] = acc[j][b];
      }
      __syncthreads();
      if (wig == 0 && lane == 0) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
          for (int b = 0; b < B; ++b) {
            float s = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < WPR; ++w2) s += red[((group * WPR + w2) * ROWS + j) * B + b];
            acc[j][b] = s;
          }
      }
    }
    if (wig == 0 && lane == 0) {
#pragma unroll
      for (int j = 0; j < ROWS; ++j) {
        const int m = m0 + j;
        if (m < M) {
#pragma unroll
          for (int b = 0; b < B; ++b)
            Y[(size_t)b * M + m] = __float2half_rn(apply_act<ACT>(acc[j][b] + bv[j]));
        }
      }
    }
    if (WPR > 1) __syncthreads();  // red[] is reused by the next pass
  }
}

struct RowdotPlan {
  int wpr, rows, grid;
};

static RowdotPlan plan_rowdot(int M, int N, int B) {
  const int sms = sm_count();
  const int nchunks = N / 8;
  const int rows = (B <= 2) ? 2 : 1;
  static const int k_wpr = env_int("DJV_RD_WPR", 0);  // development knobs
  static const int k_cap = env_int("DJV_RD_BLOCKS_PER_SM", 6);
  // As many warps per row as still lets every block be resident at once (4 blocks of 256 threads per SM):
  // a second, partial wave of blocks costs more than fewer lanes per row (measured: K=4096, d=9216 runs at
  // 0.77 of the HBM peak with 2 warps per row, 0.71 with 4, 0.67 with 1).
  const long long resident = (long long)sms * 4;
  int wpr = 1;
  while (wpr < 8 && (long long)ceil_div(M, (RD_WARPS / (wpr * 2)) * rows) <= resident && nchunks >= 64 * wpr * 2)
    wpr *= 2;
  if (k_wpr > 0) {
    wpr = k_wpr;
    while (wpr > 1 && nchunks < 32 * wpr) wpr /= 2;
  }
  const int groups = RD_WARPS / wpr;
  int grid = ceil_div(M, groups * rows);
  const int cap = sms * k_cap;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  return {wpr, rows, grid};
}

template <int B, int ACT>
static void launch_rowdot(const RowdotPlan &p, __half *Y, const __half *W, const __half *X,
                          const void *idx, const __half *bias, int M, int N, long long ldw,
                          int idx64, cudaStream_t st) {
#define DJV_RD(WPR_, ROWS_)                                                               \
  djv::launch_kernel(rowdot_kernel<B, ACT, WPR_, ROWS_, 4>, p.grid, RD_THREADS, 0, st, Y, W, X, idx, bias, M, N, \
                     ldw, idx64, (idx == nullptr || early_prefetch()) ? 1 : 0)
  constexpr int R = (B <= 2) ? 2 : 1;
  switch (p.wpr) {
    case 1: DJV_RD(1, R); break;
    case 2: DJV_RD(2, R); break;
    case 4: DJV_RD(4, R); break;
    default: DJV_RD(8, R); break;
  }
#undef DJV_RD
}

template <int B>
static int dispatch_act(const RowdotPlan &p, int act, __half *Y, const __half *W, const __half *X,
                        const void *idx, const __half *bias, int M, int N, long long ldw, int idx64,
                        cudaStream_t st) {
  switch (act) {
    case DJV_ACT_ID: launch_rowdot<B, DJV_ACT_ID>(p, Y, W, X, idx, bias, M, N, ldw, idx64, st); break;
    case DJV_ACT_RELU: launch_rowdot<B, DJV_ACT_RELU>(p, Y, W, X, idx, bias, M, N, ldw, idx64, st); break;
    case DJV_ACT_GELU: launch_rowdot<B, DJV_ACT_GELU>(p, Y, W, X, idx, bias, M, N, ldw, idx64, st); break;
    case DJV_ACT_GELU_APPROX:
      launch_rowdot<B, DJV_ACT_GELU_APPROX>(p, Y, W, X, idx, bias, M, N, ldw, idx64, st);
      break;
    case DJV_ACT_SQUARED_RELU:
      launch_rowdot<B, DJV_ACT_SQUARED_RELU>(p, Y, W, X, idx, bias, M, N, ldw, idx64, st);
      break;
    default: set_error("gather_gemv: unknown activation %d", act); return DJV_ERR_INVALID;
  }
  return DJV_OK;
}

// One launch handles up to 8 rows of x; larger batches are cut into slices of <= 8 rows
// (each slice re-reads the gathered rows).
static int rowdot_slice(int B, int act, __half *Y, const __half *W, const __half *X, const void *idx,
                        const __half *bias, int M, int N, long long ldw, int idx64, cudaStream_t st) {
  const RowdotPlan p = plan_rowdot(M, N, B);
  switch (B) {
    case 1: return dispatch_act<1>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 2: return dispatch_act<2>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 3: return dispatch_act<3>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 4: return dispatch_act<4>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 5: return dispatch_act<5>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 6: return dispatch_act<6>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 7: return dispatch_act<7>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
    case 8: return dispatch_act<8>(p, act, Y, W, X, idx, bias, M, N, ldw, idx64, st);
  }
  set_error("gather_gemv: internal batch slice %d", B);
  return DJV_ERR_INVALID;
}

// Zero rows selected (M == 0): y = bias (or 0).
__global__ void bias_fill_kernel(__half *Y, const __half *bias, int B, int N) {
  pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B * N) Y[i] = bias ? bias[i % N] : __float2half(0.f);
}

// y[n] = sum over b of x[b, n], added in fp32 in row order, rounded once
__global__ void batch_sum_kernel(__half *__restrict__ Y, const __half *__restrict__ X, int B, int N) {
  pdl_prologue();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float s = 0.f;
  for (int b = 0; b < B; ++b) s += __half2float(X[(size_t)b * N + n]);
  Y[n] = __float2half_rn(s);
}

}  // namespace djv

using namespace djv;

extern "C" int djv_batch_sum(void *y, const void *x, int B, int N, void *stream) {
  DJV_REQUIRE(y && x, "batch_sum: null pointer");
  DJV_REQUIRE(B >= 1 && N >= 1, "batch_sum: B=%d N=%d", B, N);
  djv::launch_kernel(batch_sum_kernel, ceil_div(N, 256), 256, 0, static_cast<cudaStream_t>(stream),
                     static_cast<__half *>(y), static_cast<const __half *>(x), B, N);
  count_launch();
  return check_launch("batch_sum");
}

static int check_common(const char *op, const void *y, const void *w, const void *x, int B, int N,
                        int M, long long ldw) {
  // with an empty index list there is nothing to read from x (and, for fc1, nothing to write)
  DJV_REQUIRE(w && (M == 0 || (y && x)), "%s: null pointer", op);
  DJV_REQUIRE(B >= 1 && B <= DJV_MAX_BATCH, "%s: batch %d outside [1,%d]", op, B, DJV_MAX_BATCH);
  DJV_REQUIRE(N >= 8 && N % 8 == 0, "%s: N=%d must be a positive multiple of 8", op, N);
  DJV_REQUIRE(M >= 0, "%s: negative M", op);
  DJV_REQUIRE(ldw >= N && ldw % 8 == 0, "%s: row stride %lld must be >= N and a multiple of 8", op, ldw);
  DJV_REQUIRE(aligned16(w), "%s: weight pointer must be 16-byte aligned", op);
  return DJV_OK;
}

extern "C" int djv_gather_gemv(void *y, const void *w, const void *x, const void *idx,
                               const void *bias, int B, int N, int M, long long ldw, int idx_is_64,
                               int act, void *stream) {
  int rc = check_common("gather_gemv", y, w, x, B, N, M, ldw);
  if (rc) return rc;
  DJV_REQUIRE(aligned16(x), "gather_gemv: x must be 16-byte aligned");
  DJV_REQUIRE(act >= DJV_ACT_ID && act <= DJV_ACT_SQUARED_RELU, "gather_gemv: unknown activation %d", act);
  if (M == 0) return DJV_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M <= ring_gemv_rows() && ring_shape_ok(B, N, M)) {
    rc = ring_fc1(static_cast<__half *>(y), static_cast<const __half *>(w), static_cast<const __half *>(x), idx,
                  static_cast<const __half *>(bias), B, N, M, ldw, idx_is_64, act, st);
    if (rc) return rc;
    return check_launch("gather_gemv");
  }
  // Enough activation rows make this a real small-N contraction: tensor cores, from 5 rows up (the kernel splits the
  // reduction over the blocks of a cluster when the index list is short); for 3 and 4 rows only when there are
  // >= 256 tiles of 16 gathered rows, below that the CUDA-core kernel wins.
  static const int k_mma_min_b = env_int("DJV_MMA_MIN_B", 3);         // development knobs
  static const int k_mma_always_b = env_int("DJV_MMA_ALWAYS_B", 5);
  static const int k_mma_min_tiles = env_int("DJV_MMA_MIN_TILES", 256);
  if (B >= k_mma_always_b || (B >= k_mma_min_b && ceil_div(M, MM_ROWS) >= k_mma_min_tiles)) {
    rc = rowdot_mma(B, act, static_cast<__half *>(y), static_cast<const __half *>(w),
                    static_cast<const __half *>(x), idx, static_cast<const __half *>(bias), M, N, ldw,
                    idx_is_64, st);
    if (rc) return rc;
    count_launch();
    return check_launch("gather_gemv");
  }
  for (int b0 = 0; b0 < B; b0 += 8) {
    const int bs = (B - b0 < 8) ? (B - b0) : 8;
    rc = rowdot_slice(bs, act, static_cast<__half *>(y) + (size_t)b0 * M, static_cast<const __half *>(w),
                      static_cast<const __half *>(x) + (size_t)b0 * N, idx,
                      static_cast<const __half *>(bias), M, N, ldw, idx_is_64, st);
    if (rc) return rc;
    count_launch();
  }
  return check_launch("gather_gemv");
}

extern "C" size_t djv_gather_transposed_gemv_scratch_bytes(int B, int N, int M) {
  if (B < 1 || N < 8 || M < 0) return 0;
  if (B > RA_MAX_B) return rowaxpy_mma_scratch_bytes(B, N, M > 0 ? M : 1);  // tensor-core kernel, one pass
  // up to 4 rows of x: the CUDA-core kernel's plan depends on the row count (and djv_gather_transposed_gemv_push
  // always runs it); 3 and 4 rows otherwise go to the tensor-core kernel
  const int bs = B < 4 ? B : 4;
  size_t need = B >= RA_MMA_MIN_B ? rowaxpy_mma_scratch_bytes(B, N, M > 0 ? M : 1) : 0;
  for (int b = 1; b <= bs; ++b) {
    const size_t n = rowaxpy_scratch_bytes(b, N, M);
    if (n > need) need = n;
  }
  return need;
}

extern "C" int djv_gather_transposed_gemv(void *y, const void *w, const void *x, const void *idx,
                                          const void *bias, int B, int N, int M, long long ldw,
                                          int idx_is_64, void *scratch, size_t scratch_bytes,
                                          void *stream) {
  int rc = check_common("gather_transposed_gemv", y, w, x, B, N, M, ldw);
  if (rc) return rc;
  DJV_REQUIRE(y != nullptr && aligned16(y), "gather_transposed_gemv: y must be non-null and 16-byte aligned");
  DJV_REQUIRE(bias == nullptr || aligned16(bias), "gather_transposed_gemv: bias must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M == 0) {
    djv::launch_kernel(bias_fill_kernel, ceil_div(B * N, 256), 256, 0, st, static_cast<__half *>(y),
                                                          static_cast<const __half *>(bias), B, N);
    count_launch();
    return check_launch("gather_transposed_gemv");
  }
  const size_t need = djv_gather_transposed_gemv_scratch_bytes(B, N, M);
  if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
    set_error("gather_transposed_gemv: scratch needs %zu bytes, 256-byte aligned (got %zu)", need,
              scratch_bytes);
    return DJV_ERR_SCRATCH;
  }
  if (M <= ring_gemv_rows() && ring_shape_ok(B, N, M) && scratch_bytes >= djv_mlp_sparse_fused_scratch_bytes(B, N, M)) {
    rc = ring_fc2(static_cast<__half *>(y), static_cast<const __half *>(w), static_cast<const __half *>(x), idx,
                  static_cast<const __half *>(bias), B, N, M, ldw, idx_is_64, scratch, st, PushTarget{});
    if (rc) return rc;
    return check_launch("gather_transposed_gemv");
  }
  if (B >= RA_MMA_MIN_B) {  // 3..32 activation rows: tensor cores, every gathered row read once
    rc = rowaxpy_mma(B, static_cast<__half *>(y), static_cast<const __half *>(w), static_cast<const __half *>(x), idx,
                     static_cast<const __half *>(bias), scratch, M, N, ldw, idx_is_64, st);
    if (rc) return rc;
    return check_launch("gather_transposed_gemv");
  }
  for (int b0 = 0; b0 < B; b0 += 4) {
    const int bs = (B - b0 < 4) ? (B - b0) : 4;
    rc = rowaxpy_slice(bs, static_cast<__half *>(y) + (size_t)b0 * N, static_cast<const __half *>(w),
                       static_cast<const __half *>(x) + (size_t)b0 * M, idx,
                       static_cast<const __half *>(bias), scratch, M, N, ldw, idx_is_64, st);
    if (rc) return rc;
    count_launch();
  }
  return check_launch("gather_transposed_gemv");
}

// fc2 with the result sent into every rank's receive buffer of the tensor-parallel exchange instead of y
// as exchange number `seq` of the step (see push.cuh); the consumer of that exchange is called with
// partial == NULL.
extern "C" int djv_gather_transposed_gemv_push(djv_comm *comm, int seq, const void *w, const void *x, const void *idx,
                                               const void *bias, int B, int N, int M, long long ldw,
                                               int idx_is_64, void *scratch, size_t scratch_bytes,
                                               void *stream) {
  DJV_REQUIRE(comm != nullptr && seq >= 0, "gather_transposed_gemv_push: null comm or negative exchange number");
  DJV_REQUIRE(M >= 1, "gather_transposed_gemv_push: needs at least one row");
  int rc = check_common("gather_transposed_gemv_push", w /* y unused */, w, x, B, N, M, ldw);
  if (rc) return rc;
  DJV_REQUIRE(B <= RA_MAX_B, "gather_transposed_gemv_push: batch %d above %d", B, RA_MAX_B);
  DJV_REQUIRE((size_t)B * N * 2 <= comm->slot_bytes, "gather_transposed_gemv_push: %zu bytes exceed the slot (%zu)",
              (size_t)B * N * 2, comm->slot_bytes);
  DJV_REQUIRE(bias == nullptr || aligned16(bias), "gather_transposed_gemv_push: bias must be 16-byte aligned");
  const size_t need = djv_gather_transposed_gemv_scratch_bytes(B, N, M);
  if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
    set_error("gather_transposed_gemv_push: scratch needs %zu bytes, 256-byte aligned (got %zu)", need, scratch_bytes);
    return DJV_ERR_SCRATCH;
  }
  rc = rowaxpy_slice(B, nullptr, static_cast<const __half *>(w), static_cast<const __half *>(x), idx,
                     static_cast<const __half *>(bias), scratch, M, N, ldw, idx_is_64,
                     static_cast<cudaStream_t>(stream), push_target(comm, seq));
  if (rc) return rc;
  count_launch();
  return check_launch("gather_transposed_gemv_push");
}

extern "C" int djv_mlp_sparse(void *y, void *h, const void *w1, const void *w2t, const void *x,
                              const void *idx, const void *bias1, const void *bias2, int B, int N,
                              int M, long long ldw1, long long ldw2t, int idx_is_64, void *scratch,
                              size_t scratch_bytes, void *stream) {
  DJV_REQUIRE(h != nullptr || M == 0, "mlp_sparse: h workspace is null");
  int rc = djv_gather_gemv(h, w1, x, idx, bias1, B, N, M, ldw1, idx_is_64, DJV_ACT_RELU, stream);
  if (rc) return rc;
  return djv_gather_transposed_gemv(y, w2t, h, idx, bias2, B, N, M, ldw2t, idx_is_64, scratch,
                                    scratch_bytes, stream);
}
