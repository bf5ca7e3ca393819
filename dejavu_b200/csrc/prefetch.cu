// L2 warm-up kernels for the tensor-parallel regime, where the weights one rank reads per layer (tens of MB)
// fit the 126 MB L2 several times over and every kernel of the decode step is bound by latency, not bandwidth:
// as soon as an index list exists (the top-K of a predictor has run, a good part of a layer before the kernels
// that use it), a tiny kernel on the side stream asks for the rows it names with bulk L2 prefetches. HBM is
// mostly idle at that point; the consumers later find their rows in L2. Prefetches are hints: they change no
// result, and an index outside the matrix is skipped.
#include "common.cuh"

namespace djv {

constexpr int PF_THREADS = 256;
constexpr unsigned PF_PIECE = 8192;  // bytes per bulk prefetch

__device__ __forceinline__ void bulk_prefetch_l2(const void *p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// rows idx[0..M) of up to 3 matrices that share the index list; a row is row_bytes contiguous bytes (a multiple
// of 16) at base + idx * ld_bytes
__global__ void __launch_bounds__(PF_THREADS)
prefetch_rows_kernel(const char *w0, const char *w1, const char *w2, const void *__restrict__ idx, int idx64, int M,
                     int zrows, long long ld_bytes, unsigned row_bytes) {
  pdl_prologue();  // the index list is complete after this
  const unsigned pieces = (row_bytes + PF_PIECE - 1) / PF_PIECE;
  const long long total = (long long)M * pieces;
  for (long long it = (long long)blockIdx.x * PF_THREADS + threadIdx.x; it < total;
       it += (long long)gridDim.x * PF_THREADS) {
    const int m = (int)(it / pieces);
    const unsigned pc = (unsigned)(it % pieces);
    const long long r = load_index(idx, m, idx64);
    if (r < 0 || r >= zrows) continue;
    const unsigned off = pc * PF_PIECE;
    const unsigned n = (row_bytes - off < PF_PIECE) ? row_bytes - off : PF_PIECE;
    const long long at = r * ld_bytes + off;
    if (w0) bulk_prefetch_l2(w0 + at, n);
    if (w1) bulk_prefetch_l2(w1 + at, n);
    if (w2) bulk_prefetch_l2(w2 + at, n);
  }
}

// segments of seg_bytes (a multiple of 128) at base + n * ld_bytes + idx[i] * seg_bytes, n < nrows, i < M: the
// columns of a (nrows, nheads, head_dim) matrix that belong to the listed heads
__global__ void __launch_bounds__(PF_THREADS)
prefetch_segments_kernel(const char *w, const int *__restrict__ idx, int M, int zrows, int nrows, long long ld_bytes,
                         unsigned seg_bytes) {
  pdl_prologue();
  const unsigned lines = seg_bytes / 128;
  const long long total = (long long)nrows * M * lines;
  for (long long it = (long long)blockIdx.x * PF_THREADS + threadIdx.x; it < total;
       it += (long long)gridDim.x * PF_THREADS) {
    const unsigned ln = (unsigned)(it % lines);
    const long long t = it / lines;
    const int i = (int)(t % M);
    const long long n = t / M;
    const int h = idx[i];
    if (h < 0 || h >= zrows) continue;
    prefetch_l2(w + n * ld_bytes + (long long)h * seg_bytes + ln * 128);
  }
}

}  // namespace djv

using namespace djv;

extern "C" int djv_prefetch_rows_l2(const void *w0, const void *w1, const void *w2, const void *idx, int idx_is_64,
                                    int M, int Z, long long ld_bytes, long long row_bytes, void *stream) {
  DJV_REQUIRE(idx != nullptr && (w0 || w1 || w2), "prefetch_rows_l2: null pointer");
  DJV_REQUIRE(M >= 0 && Z >= 1, "prefetch_rows_l2: bad M=%d Z=%d", M, Z);
  DJV_REQUIRE(row_bytes >= 16 && row_bytes % 16 == 0 && row_bytes < (1ll << 31) && ld_bytes % 16 == 0,
              "prefetch_rows_l2: row size and stride must be multiples of 16 bytes");
  DJV_REQUIRE((!w0 || aligned16(w0)) && (!w1 || aligned16(w1)) && (!w2 || aligned16(w2)),
              "prefetch_rows_l2: matrices must be 16-byte aligned");
  if (M == 0) return DJV_OK;
  const long long total = (long long)M * ((row_bytes + PF_PIECE - 1) / PF_PIECE);
  int grid = (int)((total + PF_THREADS - 1) / PF_THREADS);
  if (grid > 64) grid = 64;
  djv::launch_kernel(prefetch_rows_kernel, grid, PF_THREADS, 0, static_cast<cudaStream_t>(stream),
                     static_cast<const char *>(w0), static_cast<const char *>(w1), static_cast<const char *>(w2), idx,
                     idx_is_64, M, Z, ld_bytes, (unsigned)row_bytes);
  count_launch();
  return check_launch("prefetch_rows_l2");
}

extern "C" int djv_prefetch_segments_l2(const void *w, const int32_t *idx, int M, int Z, int nrows,
                                        long long ld_bytes, int seg_bytes, void *stream) {
  DJV_REQUIRE(w != nullptr && idx != nullptr, "prefetch_segments_l2: null pointer");
  DJV_REQUIRE(M >= 0 && Z >= 1 && nrows >= 1, "prefetch_segments_l2: bad sizes");
  DJV_REQUIRE(seg_bytes >= 128 && seg_bytes % 128 == 0, "prefetch_segments_l2: segments must be multiples of 128 bytes");
  if (M == 0) return DJV_OK;
  const long long total = (long long)nrows * M * (seg_bytes / 128);
  int grid = (int)((total + PF_THREADS - 1) / PF_THREADS);
  if (grid > 148) grid = 148;
  djv::launch_kernel(prefetch_segments_kernel, grid, PF_THREADS, 0, static_cast<cudaStream_t>(stream),
                     static_cast<const char *>(w), idx, M, Z, nrows, ld_bytes, (unsigned)seg_bytes);
  count_launch();
  return check_launch("prefetch_segments_l2");
}
