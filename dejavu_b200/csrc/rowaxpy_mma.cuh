// rowaxpy_mma: gather transposed GEMV (fc2) for 5..32 rows of x on the tensor cores, ONE pass over the gathered rows.
//
//   y[b, n] = sum_m x[b, m] * w[idx[m], n] + bias[n]
//
// With this many activation rows the CUDA-core kernel would either keep 8*B sums per lane or re-read every
// gathered row once per slice of 4 activation rows. Here the product is tiled as mma.sync m16n8k16 (fp16 in, fp32
// accumulate): M = activation rows (16 per tile, 1 or 2 tiles), K = 16 gathered rows, N = 8 columns.
// A warp owns 128 columns and walks the block's rows 16 at a time ("step"). The 16 x 256 bytes of a step go from
// global to the warp's own shared-memory ring with 16-byte asynchronous copies (cp.async), D steps deep: 16
// consecutive lanes copy the 256 contiguous bytes of one row, so every 8-lane group of a request covers one
// full 128-byte line. (Loading straight into the B-fragment layout would have the 8 lanes of such a group touch
// 4 different rows, 32 bytes each: four times the L1 requests per byte, measured at 0.2 of the HBM peak.)
// ldmatrix.trans then hands each lane the (k, k+1) pairs of its fragment column. The rows of the ring are padded
// to 272 bytes, which spreads the 8 row addresses of an ldmatrix over all banks.
// The 16 activations per activation row that multiply a step (the A fragments) travel with it: 32 bytes per
// activation row in the same ring stage, read back with ldmatrix. The row numbers of the block's rows (at most
// 1024) are staged in shared memory once, before the first copy.
// Rows are split over gridDim.y blocks; with more than one the per-block sums go to `partial` and a second small
// kernel adds them in block order (deterministic), all columns in parallel.
// Traffic: every gathered row is read once, whatever B is.
// (16 warps of 64 columns with 4-step rings, to hide the ldmatrix -> MMA chains behind more warps, was measured
// slower: 43 us against 40 at 8 activation rows and 6144 gathered rows of 12288 columns, 55 against 47 at 32 rows.)
#pragma once
#include "common.cuh"
#include "rowdot_mma.cuh"

namespace djv {

constexpr int RM_THREADS = 256;
constexpr int RM_WARPS = RM_THREADS / WARP;
constexpr int RM_WCOLS = 128;                   // columns per warp
constexpr int RM_BCOLS = RM_WARPS * RM_WCOLS;   // columns per block
constexpr int RM_NT = RM_WCOLS / 8;             // 8-column MMA tiles per warp
constexpr int RM_DEPTH1 = 5, RM_DEPTH2 = 4;     // steps in the ring of a warp, for 1 / 2 tiles of activation rows
constexpr int RM_PITCH = RM_WCOLS * 2 + 16;     // bytes between the rows of a step in shared memory
constexpr int RM_W_BYTES = 16 * RM_PITCH;       // the gathered rows of one step of one warp
constexpr int RM_A_PITCH = 48;                  // bytes between the activation rows of a step (32 used)
constexpr int RM_MAX_ROWS = 1024;               // rows per block (their row numbers are staged in shared memory)
constexpr int RM_IDX_BYTES = RM_MAX_ROWS * 4;
template <int NTM>
struct RmStage {
  static constexpr int BYTES = RM_W_BYTES + NTM * 16 * RM_A_PITCH;  // one step of one warp
};
template <int NTM, int D>
struct RmSmem {
  static constexpr size_t BYTES = RM_IDX_BYTES + (size_t)RM_WARPS * D * RmStage<NTM>::BYTES;
};

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst_smem, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// four 8x8 fp16 matrices: lane (g, t) gets elements [g][2t], [g][2t+1] of each ...
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr_smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr_smem)
               : "memory");
}
// ... or, transposed on the way, elements [2t][g], [2t+1][g]
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr_smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr_smem)
               : "memory");
}

template <int NTM, int D>  // tiles of 16 activation rows; steps in the ring
__global__ void __launch_bounds__(RM_THREADS, 1)
rowaxpy_mma_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
                   const void *__restrict__ idx, const __half *__restrict__ bias, float *__restrict__ partial,
                   int M, int N, long long ldw, int idx64, int B, int rows_per_block) {
  extern __shared__ __align__(128) unsigned char rm_smem[];
  constexpr int ST = RmStage<NTM>::BYTES;
  pdl_prologue();
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int g = lane / 4, t = lane % 4;
  const int col0 = blockIdx.x * RM_BCOLS + warp * RM_WCOLS;  // first column of this warp
  const int rs = blockIdx.y, RS = gridDim.y;
  const int m_begin = min(M, rs * rows_per_block), m_end = min(M, m_begin + rows_per_block);
  const int nrows = m_end - m_begin, nsteps = (nrows + 15) / 16;
  const unsigned short *Xh = reinterpret_cast<const unsigned short *>(X);
  int *idx_s = reinterpret_cast<int *>(rm_smem);  // row numbers of this block's rows
  const uint32_t ring =
      (uint32_t)__cvta_generic_to_shared(rm_smem) + RM_IDX_BYTES + (uint32_t)warp * (uint32_t)(D * ST);

  for (int i = tid; i < nrows; i += RM_THREADS) idx_s[i] = (int)load_index(idx, m_begin + i, idx64);

  float acc[NTM][RM_NT][4];
#pragma unroll
  for (int mt = 0; mt < NTM; ++mt)
#pragma unroll
    for (int nt = 0; nt < RM_NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mt][nt][c] = 0.f;
  __syncthreads();

  // copies: lanes 0-15 take the even rows of a step, lanes 16-31 the odd ones; a lane moves one 16-byte chunk
  const int lrow = lane >> 4, lchunk = lane & 15;
  const int lcol = col0 + lchunk * 8;  // N % 8 == 0: a chunk is inside the row or entirely outside
  const bool col_ok = lcol < N;
  // x[b, m .. m+7] can be copied 16 bytes at a time when those are aligned (m is a multiple of 8 here)
  const bool a_async = (M % 8) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
  // start the copies of step j: 16 gathered rows (zero-filled past the end of the block's rows) and, per
  // activation row, the 16 values that multiply them (2 chunks of 8)
  auto issue = [&](int j) {
    const uint32_t dst = ring + (uint32_t)(j % D) * ST;
    const int r0 = j * 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = 2 * i + lrow;
      const bool ok = r0 + k < nrows && col_ok;
      const __half *src = ok ? W + (long long)idx_s[r0 + k] * ldw + lcol : W;
      cp_async16_zfill(dst + (uint32_t)k * RM_PITCH + (uint32_t)lchunk * 16, src, ok ? 16 : 0);
    }
    if (a_async) {
#pragma unroll
      for (int i = 0; i < NTM; ++i) {
        const int q = lane + 32 * i, b = q >> 1, half = q & 1;
        const int k0 = r0 + half * 8;
        int bytes = (nrows - k0) * 2;
        bytes = (b < B) ? max(0, min(16, bytes)) : 0;
        const __half *src = bytes > 0 ? X + (size_t)b * M + m_begin + k0 : X;
        cp_async16_zfill(dst + RM_W_BYTES + (uint32_t)b * RM_A_PITCH + (uint32_t)half * 16, src, bytes);
      }
    }
    cp_async_commit();
  };
  // A fragments straight from x (when the 16-byte copies are not possible): x[b, m0 + k .. + 1] for
  // b = tile*16 + g (a0, a2) and + 8 (a1, a3), k = 2t (a0, a1), 2t + 8 (a2, a3)
  auto load_a = [&](int m0, uint32_t (&a)[NTM][4]) {
#pragma unroll
    for (int mt = 0; mt < NTM; ++mt) {
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int b = mt * 16 + g + (f & 1) * 8;
        const int k = m0 + 2 * t + (f >> 1) * 8;
        uint32_t v = 0;
        if (b < B && k < m_end) {
          v = Xh[(size_t)b * M + k];
          if (k + 1 < m_end) v |= (uint32_t)Xh[(size_t)b * M + k + 1] << 16;
        }
        a[mt][f] = v;
      }
    }
  };

  // prologue: steps 0 .. D-2 in flight (a commit group per step, empty of data past the last step)
#pragma unroll
  for (int j = 0; j < D - 1; ++j) issue(j);
  // ldmatrix addresses. B fragments: lane l -> row l % 16 of the step, columns (l / 16) * 8 .. + 7 of a pair of
  // tiles. A fragments: matrix i = l / 8 -> activation rows (i & 1) * 8 + l % 8, k (i / 2) * 8 .. + 7.
  const uint32_t ldb_off = (uint32_t)(lane & 15) * RM_PITCH + (uint32_t)(lane >> 4) * 16;
  const uint32_t lda_off =
      RM_W_BYTES + (uint32_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * RM_A_PITCH + (uint32_t)(lane >> 4) * 16;
  for (int s = 0; s < nsteps; ++s) {
    cp_async_wait<D - 2>();  // this lane's copies of step s have landed ...
    __syncwarp();            // ... and so have the other lanes'; all lanes are done reading step s - 1
    issue(s + D - 1);        // into the stage step s - 1 used
    const uint32_t stage = ring + (uint32_t)(s % D) * ST;
    uint32_t a[NTM][4];
    if (a_async) {
#pragma unroll
      for (int mt = 0; mt < NTM; ++mt) ldmatrix_x4(a[mt], stage + lda_off + (uint32_t)mt * 16 * RM_A_PITCH);
    } else {
      load_a(m_begin + s * 16, a);
    }
#pragma unroll
    for (int p = 0; p < RM_NT / 2; ++p) {
      uint32_t bf[4];  // b0, b1 of tile 2p; b0, b1 of tile 2p + 1
      ldmatrix_x4_trans(bf, stage + ldb_off + (uint32_t)p * 32);
#pragma unroll
      for (int mt = 0; mt < NTM; ++mt) {
        mma_m16n8k16(acc[mt][2 * p], a[mt][0], a[mt][1], a[mt][2], a[mt][3], bf[0], bf[1]);
        mma_m16n8k16(acc[mt][2 * p + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], bf[2], bf[3]);
      }
    }
  }
  cp_async_wait<0>();

  // acc[mt][nt][c]: activation row mt*16 + g (c 0,1) or + 8 (c 2,3); columns col0 + nt*8 + 2t, + 1 (c & 1)
#pragma unroll
  for (int mt = 0; mt < NTM; ++mt)
#pragma unroll
    for (int nt = 0; nt < RM_NT; ++nt)
#pragma unroll
      for (int hp = 0; hp < 2; ++hp) {
        const int b = mt * 16 + g + hp * 8, n = col0 + nt * 8 + 2 * t;  // n even, N even: the pair is inside or outside
        if (b >= B || n >= N) continue;
        float v0 = acc[mt][nt][2 * hp], v1 = acc[mt][nt][2 * hp + 1];
        if (RS == 1) {
          if (bias != nullptr) {
            const float2 bb = __half22float2(*reinterpret_cast<const __half2 *>(bias + n));
            v0 += bb.x;
            v1 += bb.y;
          }
          *reinterpret_cast<__half2 *>(Y + (size_t)b * N + n) = __floats2half2_rn(v0, v1);
        } else {
          __stcg(reinterpret_cast<float2 *>(partial + ((size_t)rs * B + b) * N + n), make_float2(v0, v1));
        }
      }
}

// y[b, n] = sum over the row blocks of partial[k][b][n] + bias[n] (deterministic). A block takes 256 columns of one
// activation row: lane l of every warp owns 8 of them, warp w adds the row blocks w, w + 8, ... in order (up to 4
// requested at a time), then the 8 warps' sums are added in warp order through shared memory.
constexpr int RM_RED_WARPS = 8;
__global__ void __launch_bounds__(RM_RED_WARPS * WARP)
rowaxpy_mma_reduce_kernel(__half *__restrict__ Y, const float *__restrict__ partial, const __half *__restrict__ bias,
                          int B, int N, int RS) {
  pdl_prologue();
  __shared__ float red[RM_RED_WARPS][WARP][8];
  const int lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
  const int b = blockIdx.y, n = (blockIdx.x * WARP + lane) * 8;
  const bool inside = n < N;  // N % 8 == 0
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  if (inside) {
    for (int k0 = warp; k0 < RS; k0 += RM_RED_WARPS * 4) {
      float4 lo[4], hi[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * RM_RED_WARPS;
        if (k < RS) {
          const float4 *src = reinterpret_cast<const float4 *>(partial + ((size_t)k * B + b) * N + n);
          lo[u] = __ldcg(src);
          hi[u] = __ldcg(src + 1);
        } else {
          lo[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          hi[u] = lo[u];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[0] += lo[u].x; v[1] += lo[u].y; v[2] += lo[u].z; v[3] += lo[u].w;
        v[4] += hi[u].x; v[5] += hi[u].y; v[6] += hi[u].z; v[7] += hi[u].w;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[warp][lane][e] = v[e];
  __syncthreads();
  if (warp != 0 || !inside) return;
#pragma unroll
  for (int w = 1; w < RM_RED_WARPS; ++w)
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] += red[w][lane][e];
  if (bias != nullptr) {
    const uint4 bv = ld_cached16(bias + n);
    const float2 b0 = h2f(bv.x), b1 = h2f(bv.y), b2 = h2f(bv.z), b3 = h2f(bv.w);
    v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y; v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
  }
  __half2 out[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) out[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4 *>(Y + (size_t)b * N + n) = *reinterpret_cast<uint4 *>(out);
}

struct RowaxpyMmaPlan {
  int tiles, rs, rows_per_block;
};

inline RowaxpyMmaPlan plan_rowaxpy_mma(int M, int N) {
  const int tiles = ceil_div(N, RM_BCOLS);
  // One block per multiprocessor (the rings of its 8 warps fill the shared memory), at least 32 rows per
  // block, rows in steps of 16. Few row blocks also keep the fp32 partial sums (rs * B * N * 4 bytes, written and
  // read once) small beside the gathered rows (M * N * 2 bytes).
  int rs = sm_count() / tiles;
  const int max_rs = M / 32 > 1 ? M / 32 : 1;
  if (rs > max_rs) rs = max_rs;
  if (rs < 1) rs = 1;
  const int min_rs = ceil_div(M, RM_MAX_ROWS);
  if (rs < min_rs) rs = min_rs;
  int rpb = ceil_div(ceil_div(M, rs), 16) * 16;  // <= RM_MAX_ROWS (a multiple of 16)
  rs = ceil_div(M, rpb);
  return {tiles, rs, rpb};
}

inline size_t rowaxpy_mma_scratch_bytes(int B, int N, int M) {
  const RowaxpyMmaPlan p = plan_rowaxpy_mma(M, N);
  return 4096 + (p.rs > 1 ? (size_t)p.rs * B * N * sizeof(float) : 0);
}

// 1 <= B <= 32 (used from 3 rows up)
inline int rowaxpy_mma(int B, __half *Y, const __half *W, const __half *X, const void *idx, const __half *bias,
                       void *scratch, int M, int N, long long ldw, int idx64, cudaStream_t st) {
  const RowaxpyMmaPlan p = plan_rowaxpy_mma(M, N);
  float *partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + 4096);  // (header: other kernels' counters)
  const dim3 grid(p.tiles, p.rs);
  constexpr size_t smem1 = RmSmem<1, RM_DEPTH1>::BYTES, smem2 = RmSmem<2, RM_DEPTH2>::BYTES;
  static_assert(smem1 <= 227 * 1024 && smem2 <= 227 * 1024, "shared memory of a block");
  static const int prepared = [] {
    cudaError_t e1 = cudaFuncSetAttribute(rowaxpy_mma_kernel<1, RM_DEPTH1>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    cudaError_t e2 = cudaFuncSetAttribute(rowaxpy_mma_kernel<2, RM_DEPTH2>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e1 != cudaSuccess || e2 != cudaSuccess) cudaGetLastError();
    return (e1 == cudaSuccess && e2 == cudaSuccess) ? 0 : 1;
  }();
  if (prepared != 0) return DJV_ERR_CUDA;
  if (B <= 16)
    djv::launch_kernel(rowaxpy_mma_kernel<1, RM_DEPTH1>, grid, dim3(RM_THREADS), smem1, st, Y, W, X, idx, bias,
                       partial, M, N, ldw, idx64, B, p.rows_per_block);
  else
    djv::launch_kernel(rowaxpy_mma_kernel<2, RM_DEPTH2>, grid, dim3(RM_THREADS), smem2, st, Y, W, X, idx, bias,
                       partial, M, N, ldw, idx64, B, p.rows_per_block);
  count_launch();
  if (p.rs > 1) {
    djv::launch_kernel(rowaxpy_mma_reduce_kernel, dim3(ceil_div(N / 8, WARP), B), dim3(RM_RED_WARPS * WARP), 0, st, Y,
                       static_cast<const float *>(partial), bias, B, N, p.rs);
    count_launch();
  }
  return DJV_OK;
}

}  // namespace djv
