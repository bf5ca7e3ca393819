// Device helpers shared by the residual+LayerNorm kernel and the all-reduce epilogue.
#pragma once
#include "common.cuh"

namespace djv {

constexpr int LN_THREADS = 512;
constexpr int LN_MAX_CHUNKS = 8;  // 16-byte chunks per thread kept in registers -> d <= 32768
// kernels are instantiated for 2, 4 and 8 chunks per thread (d <= 8192, 16384, 32768)
#define DJV_LN_DISPATCH(nchunks, CALL)            \
  do {                                            \
    if ((nchunks) <= 2 * LN_THREADS) { CALL(2); } \
    else if ((nchunks) <= 4 * LN_THREADS) { CALL(4); } \
    else { CALL(8); }                             \
  } while (0)

__device__ __forceinline__ float block_sum(float v, float *red) {
  const int lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < LN_THREADS / WARP) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// gamma and beta chunks of this thread. They are weights, not produced by any kernel of the step, so a kernel
// may fetch them before it waits for its predecessors (between griddepcontrol.launch_dependents and .wait).
template <int NCH>
struct LnAffine {
  uint4 g[NCH], b[NCH];
};
template <int NCH>
__device__ __forceinline__ void ln_fetch_affine(LnAffine<NCH> &w, const __half *gamma, const __half *beta,
                                                int nchunks) {
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int ch = c * LN_THREADS + threadIdx.x;
    if (ch < nchunks) {
      w.g[c] = ld_cached16(gamma + (size_t)ch * 8);
      w.b[c] = ld_cached16(beta + (size_t)ch * 8);
    } else {
      w.g[c] = make_uint4(0, 0, 0, 0);
      w.b[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Shared by the plain kernel and the all-reduce epilogue: normalise the fp32 values a thread holds.
// vals[c][e] belong to chunk (c*LN_THREADS + tid); chunks beyond nchunks hold zeros and are not stored.
// y2_row: optional second destination of the same row.
template <int NCH>
__device__ __forceinline__ void layernorm_store(float (&vals)[NCH][8], int nchunks, int d,
                                                const LnAffine<NCH> &w, float eps, __half *y_row, float *red,
                                                __half *y2_row = nullptr) {
  const int tid = threadIdx.x;
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e) s += vals[c][e];
  const float mean = block_sum(s, red) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    if (c * LN_THREADS + tid < nchunks) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float t = vals[c][e] - mean;
        q += t * t;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / (float)d + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int ch = c * LN_THREADS + tid;
    if (ch < nchunks) {
      const uint4 gv = w.g[c], bv = w.b[c];
      const float2 g0 = h2f(gv.x), g1 = h2f(gv.y), g2 = h2f(gv.z), g3 = h2f(gv.w);
      const float2 b0 = h2f(bv.x), b1 = h2f(bv.y), b2 = h2f(bv.z), b3 = h2f(bv.w);
      __half2 o[4];
      o[0] = __floats2half2_rn((vals[c][0] - mean) * rstd * g0.x + b0.x, (vals[c][1] - mean) * rstd * g0.y + b0.y);
      o[1] = __floats2half2_rn((vals[c][2] - mean) * rstd * g1.x + b1.x, (vals[c][3] - mean) * rstd * g1.y + b1.y);
      o[2] = __floats2half2_rn((vals[c][4] - mean) * rstd * g2.x + b2.x, (vals[c][5] - mean) * rstd * g2.y + b2.y);
      o[3] = __floats2half2_rn((vals[c][6] - mean) * rstd * g3.x + b3.x, (vals[c][7] - mean) * rstd * g3.y + b3.y);
      *reinterpret_cast<uint4 *>(y_row + (size_t)ch * 8) = *reinterpret_cast<uint4 *>(o);
      if (y2_row) *reinterpret_cast<uint4 *>(y2_row + (size_t)ch * 8) = *reinterpret_cast<uint4 *>(o);
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
  const float2 a = h2f(v.x), b = h2f(v.y), c = h2f(v.z), d = h2f(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// round 8 fp32 values to fp16, store them, and keep the rounded values
__device__ __forceinline__ void round_store8(float (&f)[8], __half *dst) {
  __half2 o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) o[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
  if (dst) *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<uint4 *>(o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 t = __half22float2(o[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}

}  // namespace djv
