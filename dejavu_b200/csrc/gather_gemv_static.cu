// djv_gather_transposed_gemv_static — the gather transposed GEMV (fc2) for callers that cannot hand the
// library any scratch memory of their own.
//
// Who that is: a host that gave all of the GPU's memory to its own pool at start-up and has nothing left
// to cudaMalloc; a plugin called from inside a region where allocation is forbidden (a stream being
// captured into a CUDA graph, a real-time loop that must not take the allocator's implicit
// synchronisation); a binding layer with no notion of workspace buffers at all. The regular entry point
// (djv_gather_transposed_gemv) asks such callers for something they cannot give.
//
// Here the scratch (block counters + per-cluster partial sums) lives in ONE file-scope __device__ array of
// DJV_STATIC_SCRATCH_BYTES, which every GPU that loads this library holds until the process exits. The
// array's name is only a host-side handle: the device address is looked up once per device with
// cudaGetSymbolAddress (checked) on the first call made while that device is current, and that address is
// what the kernel receives. That first call performs the lookup, so make it before any stream capture
// begins. Nothing in this file calls cudaMalloc, cudaFree or any allocating library routine.
//
// All calls on a device share the array and it keeps whatever the last call left behind. The counter
// words, which must start at zero, are cleared on the caller's stream before every launch; the partial
// sums are fully overwritten before they are read. Two calls that overlap on the GPU (different streams
// without an ordering between them, or two host threads) race on the array: order them.
#include <mutex>

#include "rowaxpy.cuh"

namespace djv {

static __device__ __align__(256) unsigned char g_static_scratch[DJV_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static void *g_scratch_addr[MAX_DEVICES];
static std::mutex g_scratch_mutex;

// Device address of g_static_scratch on the current device, resolved once per device.
static int static_scratch(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_error("gather_transposed_gemv_static: cannot identify the current device (%s)",
              e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("gather_transposed_gemv_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                cudaGetErrorString(e));
      return DJV_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DJV_OK;
}

}  // namespace djv

using namespace djv;

extern "C" int djv_gather_transposed_gemv_static(void *y, const void *w, const void *x, const void *idx,
                                                 const void *bias, int B, int N, int M, long long ldw,
                                                 int idx_is_64, void *stream) {
  DJV_REQUIRE(y && w && (M == 0 || x), "gather_transposed_gemv_static: null pointer");
  DJV_REQUIRE(B >= 1 && B <= RA_MAX_B, "gather_transposed_gemv_static: batch %d outside [1,%d]", B, RA_MAX_B);
  DJV_REQUIRE(N >= 8 && N % 8 == 0, "gather_transposed_gemv_static: N=%d must be a positive multiple of 8", N);
  DJV_REQUIRE(M >= 1, "gather_transposed_gemv_static: M=%d must be at least 1", M);
  DJV_REQUIRE(ldw >= N && ldw % 8 == 0, "gather_transposed_gemv_static: bad row stride %lld", ldw);
  DJV_REQUIRE(aligned16(w), "gather_transposed_gemv_static: weight pointer must be 16-byte aligned");
  // the finishing stage stores 16 bytes at a time to y and loads 16 bytes at a time from bias
  DJV_REQUIRE(aligned16(y), "gather_transposed_gemv_static: y must be 16-byte aligned");
  DJV_REQUIRE(bias == nullptr || aligned16(bias), "gather_transposed_gemv_static: bias must be 16-byte aligned");
  const size_t need = rowaxpy_scratch_bytes(B, N, M);
  if (need > DJV_STATIC_SCRATCH_BYTES) {
    set_error("gather_transposed_gemv_static: B=%d N=%d M=%d needs %zu bytes of scratch, the built-in array holds "
              "%u; use djv_gather_transposed_gemv with caller-provided scratch",
              B, N, M, need, (unsigned)DJV_STATIC_SCRATCH_BYTES);
    return DJV_ERR_SCRATCH;
  }
  void *scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the counters must start at zero whatever an earlier (possibly aborted) call left there
  cudaError_t e = cudaMemsetAsync(scratch, 0, RA_COUNTER_BYTES, st);
  if (e != cudaSuccess) {
    set_error("gather_transposed_gemv_static: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  rc = rowaxpy_slice(B, static_cast<__half *>(y), static_cast<const __half *>(w),
                     static_cast<const __half *>(x), idx, static_cast<const __half *>(bias), scratch, M, N, ldw,
                     idx_is_64, st);
  if (rc) return rc;
  count_launch();
  return check_launch("gather_transposed_gemv_static");
}
