// Residual add + LayerNorm for the decode step (one block per token row).
//   r = fp16(x + residual + xbias);  y = fp16((r - mean) * rstd * gamma + beta)
// Statistics are taken in fp32 over the fp16-rounded r, which is what an fp16 add followed by
// torch.nn.LayerNorm computes. Bytes: 3 reads + 2 writes of d fp16 per row (+ gamma, beta).
#include "norm.cuh"

namespace djv {

template <int NCH>
__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_kernel(__half *__restrict__ y, __half *r_out, const __half *__restrict__ x,
                     const __half *residual, const __half *__restrict__ xbias,
                     const __half *__restrict__ gamma, const __half *__restrict__ beta, int d, float eps) {
  __shared__ float red[LN_THREADS / WARP];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int nchunks = d / 8;
  // the affine weights are fetched while the predecessor kernel may still be running
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  LnAffine<NCH> w;
  ln_fetch_affine(w, gamma, beta, nchunks);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const size_t off = (size_t)row * d;
  float vals[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int ch = c * LN_THREADS + tid;
    if (ch < nchunks) {
      float f[8], t[8];
      unpack8(ld_cached16(x + off + (size_t)ch * 8), f);
      if (residual) {
        unpack8(*reinterpret_cast<const uint4 *>(residual + off + (size_t)ch * 8), t);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += t[e];
      }
      if (xbias) {
        unpack8(ld_cached16(xbias + (size_t)ch * 8), t);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += t[e];
      }
      round_store8(f, r_out ? r_out + off + (size_t)ch * 8 : nullptr);
#pragma unroll
      for (int e = 0; e < 8; ++e) vals[c][e] = f[e];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) vals[c][e] = 0.f;
    }
  }
  layernorm_store(vals, nchunks, d, w, eps, y + off, red);
}

}  // namespace djv

using namespace djv;

extern "C" int djv_add_layernorm(void *y, void *r_out, const void *x, const void *residual,
                                 const void *xbias, const void *gamma, const void *beta, int B, int d,
                                 float eps, void *stream) {
  DJV_REQUIRE(y && x && gamma && beta, "add_layernorm: null pointer");
  DJV_REQUIRE(B >= 1, "add_layernorm: batch %d", B);
  DJV_REQUIRE(d >= 8 && d % 8 == 0 && d / 8 <= LN_THREADS * LN_MAX_CHUNKS,
              "add_layernorm: d=%d must be a multiple of 8 and <= %d", d, LN_THREADS * LN_MAX_CHUNKS * 8);
  DJV_REQUIRE(aligned16(y) && aligned16(x) && aligned16(gamma) && aligned16(beta) &&
                  (!r_out || aligned16(r_out)) && (!residual || aligned16(residual)) &&
                  (!xbias || aligned16(xbias)),
              "add_layernorm: pointers must be 16-byte aligned");
#define DJV_LN_CALL(NCH_)                                                                                      \
  djv::launch_kernel(add_layernorm_kernel<NCH_>, B, LN_THREADS, 0, static_cast<cudaStream_t>(stream),          \
                     static_cast<__half *>(y), static_cast<__half *>(r_out), static_cast<const __half *>(x),  \
                     static_cast<const __half *>(residual), static_cast<const __half *>(xbias),               \
                     static_cast<const __half *>(gamma), static_cast<const __half *>(beta), d, eps)
  DJV_LN_DISPATCH(d / 8, DJV_LN_CALL);
#undef DJV_LN_CALL
  count_launch();
  return check_launch("add_layernorm");
}
