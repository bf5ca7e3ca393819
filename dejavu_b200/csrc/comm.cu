// Tensor-parallel one-shot all-reduce fused with the residual add and LayerNorm that follow it.
//
// Push protocol, the data is its own arrival flag: every rank owns a receive buffer of
// 3 slots x world pieces, mapped into every peer with CUDA IPC and filled with a sentinel (fp16 -0.0,
// bits 0x8000). One call = one block per rank, step e uses slot e % 3:
//   1. each thread stores its 16-byte chunks of this rank's partial into piece [rank] of slot e%3 of EVERY
//      rank (plain stores over NVLink; -0.0 in the data is sent as +0.0, which changes no sum);
//   2. each thread refills slot (e+2)%3 of the LOCAL buffer with the sentinel. That slot held step e-1,
//      which this rank finished reading before it started step e, and no peer writes it again before step
//      e+2, which a peer can only reach after this rank's step e+1 push, i.e. after this kernel ended;
//   3. each thread polls (bounded) the same chunks of all pieces of the LOCAL slot e%3 until no half of a
//      chunk is the sentinel, adds them in rank order in fp32 (same order on all ranks, so all ranks hold
//      bit-identical results), rounds to fp16, adds the residual, and the block normalises.
// One NVLink one-way trip per step, no fences, no remote loads. A 16-byte store may arrive in pieces: every
// half of a chunk is checked, so a partly arrived chunk just keeps the thread polling.
// The epoch lives in device memory and is advanced by the kernel, so a captured CUDA graph replays correctly.
// No multicast / multimem objects are used: a peer that exits between steps cannot fault the others,
// their next call just runs out its wait and reports DJV_ERR_TIMEOUT in the status word.
#include "norm.cuh"
#include "push.cuh"

namespace djv {

constexpr unsigned long long AR_WAIT_LIMIT_NS = 2000ull * 1000 * 1000;  // a wait on a peer gives up after 2 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void fill_sentinel_kernel(uint4 *p, size_t n16) {
  const uint4 s = make_uint4(AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
    p[i] = s;
}

template <int NCH>
__global__ void __launch_bounds__(LN_THREADS)
allreduce_add_layernorm_kernel(void *const *__restrict__ bufs, unsigned *__restrict__ epoch_status, int rank,
                               int world, size_t slot_bytes, __half *__restrict__ y, __half *r_out,
                               const __half *__restrict__ partial, const __half *residual,
                               const __half *__restrict__ gamma, const __half *__restrict__ beta,
                               int B, int d, float eps) {
  __shared__ float red[LN_THREADS / WARP];
  __shared__ int failed;
  const int tid = threadIdx.x;
  const int nchunks = d / 8;
  // the affine weights are fetched while the predecessor kernel may still be running
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  LnAffine<NCH> w;
  ln_fetch_affine(w, gamma, beta, nchunks);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned epoch = epoch_status[0];
  const int total_chunks = B * nchunks;
  if (tid == 0) failed = 0;
  // once a wait has run out the exchange is dead: later calls return at once instead of waiting again
  if (epoch_status[1] != 0u) return;
  __syncthreads();
  const size_t cur_off = (size_t)(epoch % AR_SLOTS) * world * slot_bytes;
  const size_t old_off = (size_t)((epoch + 2) % AR_SLOTS) * world * slot_bytes;

  // 1. push this rank's partial into piece [rank] of the current slot of every rank
  //    (partial == nullptr: the kernel that produced it has pushed it already, see push.cuh)
  if (partial != nullptr) {
    void *dst[AR_MAX_WORLD];
#pragma unroll
    for (int p = 0; p < AR_MAX_WORLD; ++p)
      dst[p] = (p < world) ? static_cast<char *>(bufs[p]) + cur_off + (size_t)rank * slot_bytes : nullptr;
    const uint4 *src = reinterpret_cast<const uint4 *>(partial);
    for (int c = tid; c < total_chunks; c += LN_THREADS) {
      uint4 v = src[c];
      v.x = no_sentinel2(v.x); v.y = no_sentinel2(v.y); v.z = no_sentinel2(v.z); v.w = no_sentinel2(v.w);
#pragma unroll
      for (int p = 0; p < AR_MAX_WORLD; ++p)
        if (p < world) st_sys16(static_cast<uint4 *>(dst[p]) + c, v);
    }
  }
  // 2. the slot of the previous step becomes free again
  char *local = static_cast<char *>(bufs[rank]);
  {
    const uint4 s = make_uint4(AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2);
    for (int p = 0; p < world; ++p) {
      uint4 *old_piece = reinterpret_cast<uint4 *>(local + old_off + (size_t)p * slot_bytes);
      for (int c = tid; c < total_chunks; c += LN_THREADS) old_piece[c] = s;
    }
  }

  // 3. wait for the same chunks of every piece, reduce in rank order, residual add, LayerNorm
  const unsigned long long t_start = global_timer_ns();
  bool gave_up = false;
  for (int row = 0; row < B; ++row) {
    const size_t off = (size_t)row * d;
    float vals[NCH][8];
    // the residual row is requested before the wait on the peers, not after it
    uint4 rres[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int ch = c * LN_THREADS + tid;
      rres[c] = (residual && ch < nchunks) ? *reinterpret_cast<const uint4 *>(residual + off + (size_t)ch * 8)
                                           : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int ch = c * LN_THREADS + tid;
      if (ch < nchunks && !gave_up) {
        const char *piece0 = local + cur_off + (off + (size_t)ch * 8) * 2;
        uint4 v[AR_MAX_WORLD];
        unsigned missing = (1u << world) - 1u;
        // all pieces are requested together; only the ones not there yet are asked for again
        while (missing != 0u) {
#pragma unroll
          for (int p = 0; p < AR_MAX_WORLD; ++p)
            if (missing >> p & 1u) v[p] = ld_sys16(piece0 + (size_t)p * slot_bytes);
#pragma unroll
          for (int p = 0; p < AR_MAX_WORLD; ++p)
            if ((missing >> p & 1u) && arrived16(v[p])) missing &= ~(1u << p);
          if (missing != 0u && global_timer_ns() - t_start > AR_WAIT_LIMIT_NS) {
            gave_up = true;
            break;
          }
        }
        float f[8], t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = 0.f;
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p) {  // rank order
          if (p < world && !gave_up) {
            unpack8(v[p], t);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] += t[e];
          }
        }
        round_store8(f, nullptr);  // the all-reduced activation is an fp16 tensor
        if (residual) {
          unpack8(rres[c], t);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] += t[e];
        }
        if (!gave_up) round_store8(f, r_out ? r_out + off + (size_t)ch * 8 : nullptr);
#pragma unroll
        for (int e = 0; e < 8; ++e) vals[c][e] = f[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) vals[c][e] = 0.f;
      }
    }
    if (gave_up) failed = 1;
    __syncthreads();
    if (failed) break;  // block-uniform
    layernorm_store(vals, nchunks, d, w, eps, y + off, red);
  }
  if (tid == 0) {
    if (failed) epoch_status[1] = (unsigned)DJV_ERR_TIMEOUT;
    epoch_status[0] = epoch + 1;
  }
}

}  // namespace djv

using namespace djv;

extern "C" int djv_ipc_alloc(size_t bytes, void **dev_ptr_out) {
  DJV_REQUIRE(dev_ptr_out && bytes > 0, "ipc_alloc: bad argument");
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("ipc_alloc: %s", cudaGetErrorString(e));
    if (p) cudaFree(p);
    return DJV_ERR_CUDA;
  }
  *dev_ptr_out = p;
  return DJV_OK;
}

extern "C" int djv_ipc_free(void *dev_ptr) {
  if (dev_ptr && cudaFree(dev_ptr) != cudaSuccess) {
    set_error("ipc_free: cudaFree failed");
    return DJV_ERR_CUDA;
  }
  return DJV_OK;
}

extern "C" int djv_ipc_get_handle(const void *dev_ptr, unsigned char handle_out[64]) {
  DJV_REQUIRE(dev_ptr && handle_out, "ipc_get_handle: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr));
  if (e != cudaSuccess) {
    set_error("ipc_get_handle: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  memcpy(handle_out, &h, 64);
  return DJV_OK;
}

extern "C" int djv_ipc_open(const unsigned char handle[64], void **dev_ptr_out) {
  DJV_REQUIRE(handle && dev_ptr_out, "ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("ipc_open: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  return DJV_OK;
}

extern "C" int djv_ipc_close(void *dev_ptr) {
  if (!dev_ptr) return DJV_OK;
  cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
  if (e != cudaSuccess) {
    set_error("ipc_close: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  return DJV_OK;
}

extern "C" size_t djv_comm_buffer_bytes(int world, size_t slot_bytes) {
  if (world < 1 || world > AR_MAX_WORLD) return 0;
  return (size_t)AR_SLOTS * world * slot_bytes;
}

// Set-up call: allocates two small device tables with cudaMalloc, fills this rank's own receive buffer with
// the sentinel and synchronises the device. Peers must not run a step before every rank has returned from
// this call (the host puts a barrier after it).
extern "C" int djv_comm_create(djv_comm **out, int rank, int world, void *const *bufs, size_t slot_bytes) {
  DJV_REQUIRE(out && bufs, "comm_create: null pointer");
  DJV_REQUIRE(world >= 1 && world <= AR_MAX_WORLD && rank >= 0 && rank < world,
              "comm_create: rank %d / world %d (max %d)", rank, world, AR_MAX_WORLD);
  DJV_REQUIRE(slot_bytes >= 16 && slot_bytes % 256 == 0, "comm_create: slot_bytes must be a multiple of 256");
  for (int r = 0; r < world; ++r)
    DJV_REQUIRE(bufs[r] && aligned16(bufs[r]), "comm_create: rank %d buffer missing", r);
  djv_comm *c = new djv_comm();
  c->rank = rank; c->world = world; c->slot_bytes = slot_bytes;
  c->last_stream = nullptr;
  cudaError_t e = cudaMalloc(&c->bufs_dev, sizeof(void *) * AR_MAX_WORLD);
  if (e == cudaSuccess) e = cudaMalloc(&c->epoch_dev, 2 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemcpy(c->bufs_dev, bufs, sizeof(void *) * world, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(c->epoch_dev, 0, 2 * sizeof(unsigned));
  if (e == cudaSuccess) {
    fill_sentinel_kernel<<<64, 256>>>(static_cast<uint4 *>(bufs[rank]), djv_comm_buffer_bytes(world, slot_bytes) / 16);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("comm_create: %s", cudaGetErrorString(e));
    djv_comm_destroy(c);
    return DJV_ERR_CUDA;
  }
  *out = c;
  return DJV_OK;
}

extern "C" int djv_comm_destroy(djv_comm *c) {
  if (!c) return DJV_OK;
  if (c->bufs_dev) cudaFree(c->bufs_dev);
  if (c->epoch_dev) cudaFree(c->epoch_dev);
  delete c;
  return DJV_OK;
}

extern "C" int djv_comm_status(djv_comm *c) {
  DJV_REQUIRE(c, "comm_status: null comm");
  unsigned es[2] = {0, 0};
  cudaError_t e = cudaStreamSynchronize(c->last_stream);
  if (e == cudaSuccess) e = cudaMemcpy(es, c->epoch_dev, sizeof(es), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_error("comm_status: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  if ((int)es[1] != 0) set_error("all-reduce: a peer did not arrive within the wait limit (epoch %u)", es[0]);
  return (int)es[1];
}

extern "C" int djv_allreduce_add_layernorm(djv_comm *c, void *y, void *r_out, const void *partial,
                                           const void *residual, const void *gamma, const void *beta,
                                           int B, int d, float eps, void *stream) {
  DJV_REQUIRE(c && y && gamma && beta, "allreduce_add_layernorm: null pointer");
  DJV_REQUIRE(B >= 1 && d >= 8 && d % 8 == 0 && d / 8 <= LN_THREADS * LN_MAX_CHUNKS,
              "allreduce_add_layernorm: bad B=%d d=%d", B, d);
  DJV_REQUIRE((size_t)B * d * 2 <= c->slot_bytes, "allreduce_add_layernorm: %zu bytes exceed the slot (%zu)",
              (size_t)B * d * 2, c->slot_bytes);
  DJV_REQUIRE(aligned16(y) && (!partial || aligned16(partial)) && aligned16(gamma) && aligned16(beta) &&
                  (!r_out || aligned16(r_out)) && (!residual || aligned16(residual)),
              "allreduce_add_layernorm: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  c->last_stream = st;
#define DJV_AR_CALL(NCH_)                                                                                       \
  djv::launch_kernel(allreduce_add_layernorm_kernel<NCH_>, 1, LN_THREADS, 0, st, c->bufs_dev, c->epoch_dev,     \
                     c->rank, c->world, c->slot_bytes, static_cast<__half *>(y), static_cast<__half *>(r_out), \
                     static_cast<const __half *>(partial), static_cast<const __half *>(residual),              \
                     static_cast<const __half *>(gamma), static_cast<const __half *>(beta), B, d, eps)
  DJV_LN_DISPATCH(d / 8, DJV_AR_CALL);
#undef DJV_AR_CALL
  count_launch();
  return check_launch("allreduce_add_layernorm");
}
