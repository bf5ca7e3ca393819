// rowaxpy_mma: gather transposed GEMV (fc2) for 5..32 rows of x on the tensor cores, ONE pass over the gathered rows.
//
//   y[b, n] = sum_m x[b, m] * w[idx[m], n] + bias[n]
//
// With this many activation rows the CUDA-core kernel would either keep 8*B sums per lane or re-read every
// gathered row once per slice of 4 activation rows. Here the product is tiled as mma.sync m16n8k16 (fp16 in, fp32
// accumulate): M = activation rows (16 per tile, 1 or 2 tiles), K = 16 gathered rows, N = 8 columns.
// A warp owns 128 columns (two groups of 64) and walks the block's rows 16 at a time. Lane (g, t) (g = lane / 4,
// t = lane % 4) loads 16 contiguous bytes (8 columns, g-th chunk of the 64-column group) of rows 2t, 2t+1, 2t+8,
// 2t+9 of the 16: exactly the k positions its B fragments need, so the fragments are built in registers with
// byte permutes (pairing the same column of two rows) and nothing goes through shared memory. The e-th of the 8
// columns a lane holds feeds MMA number e of the group, whose "n" index is the chunk number g: MMA e of group j
// produces columns j*64 + n*8 + e. The 8 lanes that share t read 128 contiguous bytes of a row; the two groups of
// a warp make that 2 x 128 bytes per row and warp, 8 independent 16-byte loads in flight per lane.
// The activations of a 16-row step (A fragments) come from x directly (4 bytes per register, L1-resident).
// Rows are split over gridDim.y blocks; with more than one the per-block sums go to `partial` and a second small
// kernel adds them in block order (deterministic), all columns in parallel.
// Traffic: every gathered row is read once, whatever B is.
#pragma once
#include "common.cuh"
#include "rowdot_mma.cuh"

namespace djv {

constexpr int RM_THREADS = 256;
constexpr int RM_WARPS = RM_THREADS / WARP;
constexpr int RM_WCOLS = 128;                   // columns per warp
constexpr int RM_BCOLS = RM_WARPS * RM_WCOLS;   // columns per block
constexpr int RM_GROUPS = RM_WCOLS / 64;        // 64-column groups per warp

// same column of two rows -> one register: (lo, hi) halves of a and b
__device__ __forceinline__ uint32_t pair_lo(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x5410); }
__device__ __forceinline__ uint32_t pair_hi(uint32_t a, uint32_t b) { return __byte_perm(a, b, 0x7632); }

template <int NTM>  // tiles of 16 activation rows
__global__ void __launch_bounds__(RM_THREADS)
rowaxpy_mma_kernel(__half *__restrict__ Y, const __half *__restrict__ W, const __half *__restrict__ X,
                   const void *__restrict__ idx, const __half *__restrict__ bias, float *__restrict__ partial,
                   int M, int N, long long ldw, int idx64, int B, int rows_per_block) {
  pdl_prologue();
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int g = lane / 4, t = lane % 4;
  const int col0 = blockIdx.x * RM_BCOLS + warp * RM_WCOLS;  // first column of this warp
  const int rs = blockIdx.y, RS = gridDim.y;
  const int m_begin = min(M, rs * rows_per_block), m_end = min(M, m_begin + rows_per_block);
  const unsigned short *Xh = reinterpret_cast<const unsigned short *>(X);

  float acc[NTM][RM_GROUPS][8][4];
#pragma unroll
  for (int mt = 0; mt < NTM; ++mt)
#pragma unroll
    for (int j = 0; j < RM_GROUPS; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][j][e][c] = 0.f;

  // the 4 rows of a 16-row step this lane loads: k = 2t, 2t+1, 2t+8, 2t+9
  const int kq[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int m0 = m_begin; m0 < m_end; m0 += 16) {
    uint4 wv[RM_GROUPS][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int m = m0 + kq[q];
      const bool ok = m < m_end;
      const long long r = ok ? load_index(idx, m, idx64) : 0;
      const __half *wrow = W + r * ldw;
#pragma unroll
      for (int j = 0; j < RM_GROUPS; ++j) {
        const int c = col0 + j * 64 + g * 8;  // N % 8 == 0: a chunk is inside the row or entirely outside
        wv[j][q] = (ok && c < N) ? ld_stream16(wrow + c) : zero;
      }
    }
    // A fragments: x[b, m0 + k .. + 1] for b = tile*16 + g (a0, a2) and + 8 (a1, a3), k = 2t (a0, a1), 2t + 8 (a2, a3)
    uint32_t a[NTM][4];
#pragma unroll
    for (int mt = 0; mt < NTM; ++mt) {
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int b = mt * 16 + g + (f & 1) * 8;
        const int k = m0 + 2 * t + (f >> 1) * 8;
        uint32_t lo = 0, hi = 0;
        if (b < B) {
          if (k < m_end) lo = Xh[(size_t)b * M + k];
          if (k + 1 < m_end) hi = Xh[(size_t)b * M + k + 1];
        }
        a[mt][f] = lo | (hi << 16);
      }
    }
#pragma unroll
    for (int j = 0; j < RM_GROUPS; ++j) {
      const uint32_t r0[4] = {wv[j][0].x, wv[j][0].y, wv[j][0].z, wv[j][0].w};
      const uint32_t r1[4] = {wv[j][1].x, wv[j][1].y, wv[j][1].z, wv[j][1].w};
      const uint32_t r2[4] = {wv[j][2].x, wv[j][2].y, wv[j][2].z, wv[j][2].w};
      const uint32_t r3[4] = {wv[j][3].x, wv[j][3].y, wv[j][3].z, wv[j][3].w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t b0 = (e & 1) ? pair_hi(r0[e / 2], r1[e / 2]) : pair_lo(r0[e / 2], r1[e / 2]);
        const uint32_t b1 = (e & 1) ? pair_hi(r2[e / 2], r3[e / 2]) : pair_lo(r2[e / 2], r3[e / 2]);
#pragma unroll
        for (int mt = 0; mt < NTM; ++mt)
          mma_m16n8k16(acc[mt][j][e], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
      }
    }
  }

  // acc[mt][j][e][c]: activation row mt*16 + g (c 0,1) or + 8 (c 2,3); column col0 + j*64 + n*8 + e, n = 2t (c 0,2) or 2t+1
  auto column = [&](int j, int e, int c) { return col0 + j * 64 + (2 * t + (c & 1)) * 8 + e; };
  auto brow = [&](int mt, int c) { return mt * 16 + g + (c >> 1) * 8; };
  if (RS == 1) {
#pragma unroll
    for (int mt = 0; mt < NTM; ++mt)
#pragma unroll
      for (int j = 0; j < RM_GROUPS; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int b = brow(mt, c), n = column(j, e, c);
            if (b < B && n < N)
              Y[(size_t)b * N + n] = __float2half_rn(acc[mt][j][e][c] + (bias ? __half2float(bias[n]) : 0.f));
          }
    return;
  }
#pragma unroll
  for (int mt = 0; mt < NTM; ++mt)
#pragma unroll
    for (int j = 0; j < RM_GROUPS; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int b = brow(mt, c), n = column(j, e, c);
          if (b < B && n < N) __stcg(partial + ((size_t)rs * B + b) * N + n, acc[mt][j][e][c]);
        }
}

// y[b, n] = sum over the row blocks of partial[k][b][n] + bias[n], in block order (deterministic); a thread takes 8
// consecutive columns and requests all blocks' sums (up to 8 at a time) before it adds them.
__global__ void __launch_bounds__(256)
rowaxpy_mma_reduce_kernel(__half *__restrict__ Y, const float *__restrict__ partial, const __half *__restrict__ bias,
                          int B, int N, int RS) {
  pdl_prologue();
  const int chunks = N / 8;
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= B * chunks) return;
  const int b = o / chunks, n = (o % chunks) * 8;
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  for (int k0 = 0; k0 < RS; k0 += 8) {
    float4 lo[8], hi[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (k0 + u < RS) {
        const float4 *src = reinterpret_cast<const float4 *>(partial + ((size_t)(k0 + u) * B + b) * N + n);
        lo[u] = __ldcg(src);
        hi[u] = __ldcg(src + 1);
      } else {
        lo[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        hi[u] = lo[u];
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      v[0] += lo[u].x; v[1] += lo[u].y; v[2] += lo[u].z; v[3] += lo[u].w;
      v[4] += hi[u].x; v[5] += hi[u].y; v[6] += hi[u].z; v[7] += hi[u].w;
    }
  }
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
  // about two blocks per multiprocessor, at least 64 rows per block, rows in steps of 16
  int rs = ceil_div(2 * sm_count(), tiles);
  const int max_rs = M / 64 > 1 ? M / 64 : 1;
  if (rs > max_rs) rs = max_rs;
  if (rs < 1) rs = 1;
  int rpb = ceil_div(ceil_div(M, rs), 16) * 16;
  rs = ceil_div(M, rpb);
  return {tiles, rs, rpb};
}

inline size_t rowaxpy_mma_scratch_bytes(int B, int N, int M) {
  const RowaxpyMmaPlan p = plan_rowaxpy_mma(M, N);
  return 4096 + (p.rs > 1 ? (size_t)p.rs * B * N * sizeof(float) : 0);
}

// 5 <= B <= 32
inline int rowaxpy_mma(int B, __half *Y, const __half *W, const __half *X, const void *idx, const __half *bias,
                       void *scratch, int M, int N, long long ldw, int idx64, cudaStream_t st) {
  const RowaxpyMmaPlan p = plan_rowaxpy_mma(M, N);
  float *partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + 4096);  // (header: other kernels' counters)
  const dim3 grid(p.tiles, p.rs);
  if (B <= 16)
    djv::launch_kernel(rowaxpy_mma_kernel<1>, grid, dim3(RM_THREADS), 0, st, Y, W, X, idx, bias, partial, M, N, ldw,
                       idx64, B, p.rows_per_block);
  else
    djv::launch_kernel(rowaxpy_mma_kernel<2>, grid, dim3(RM_THREADS), 0, st, Y, W, X, idx, bias, partial, M, N, ldw,
                       idx64, B, p.rows_per_block);
  count_launch();
  if (p.rs > 1) {
    djv::launch_kernel(rowaxpy_mma_reduce_kernel, dim3(ceil_div(B * (N / 8), 256)), dim3(256), 0, st, Y,
                       static_cast<const float *>(partial), bias, B, N, p.rs);
    count_launch();
  }
  return DJV_OK;
}

}  // namespace djv
