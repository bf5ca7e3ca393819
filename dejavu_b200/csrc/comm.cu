// Tensor-parallel one-shot all-reduce fused with the residual add and LayerNorm that follow it.
//
// Each rank owns an exchange buffer (2 slots) and a flag array, both mapped into every peer with CUDA
// IPC. One call = one block per rank:
//   1. copy this rank's fp16 partial into its own slot (epoch % 2),
//   2. release-store epoch+1 into flag[rank] of every peer (plain stores over NVLink),
//   3. wait (bounded) until every peer's flag in local memory reached epoch+1,
//   4. load every rank's slot with plain peer loads, add in rank order in fp32 (same order on all
//      ranks, so all ranks hold bit-identical results), round to fp16, add the residual, LayerNorm.
// The epoch lives in device memory and is advanced by the kernel, so a captured CUDA graph replays
// correctly. Two slots suffice: a rank can only reach epoch e+2 after every peer signalled e+1, which
// a peer does after it finished reading slot e%2.
// No multicast / multimem objects are used: a peer that exits between steps cannot fault the others,
// their next call just runs out its wait and reports DJV_ERR_TIMEOUT in the status word.
#include "norm.cuh"

struct djv_comm {
  int rank, world, slots;
  size_t slot_bytes;
  // device-side tables (cudaMalloc'ed by djv_comm_create)
  void **bufs_dev;
  unsigned **flags_dev;
  unsigned *epoch_dev;  // [0] epoch, [1] status
  cudaStream_t last_stream;
};

namespace djv {

constexpr int AR_MAX_WORLD = 8;
constexpr unsigned long long AR_WAIT_LIMIT_NS = 2000ull * 1000 * 1000;  // a wait on a peer gives up after 2 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(LN_THREADS)
allreduce_add_layernorm_kernel(void *const *__restrict__ bufs, unsigned *const *__restrict__ flags,
                               unsigned *__restrict__ epoch_status, int rank, int world,
                               size_t slot_bytes, __half *__restrict__ y, __half *r_out,
                               const __half *__restrict__ partial, const __half *residual,
                               const __half *__restrict__ gamma, const __half *__restrict__ beta,
                               int B, int d, float eps) {
  pdl_prologue();
  __shared__ float red[LN_THREADS / WARP];
  __shared__ int failed;
  const int tid = threadIdx.x;
  const unsigned epoch = epoch_status[0];
  const unsigned want = epoch + 1;
  const size_t slot_off = (size_t)(epoch & 1u) * slot_bytes;
  const int nchunks = d / 8;
  const int total_chunks = B * nchunks;
  if (tid == 0) failed = 0;
  // once a wait has run out the exchange is dead: later calls return at once instead of waiting again
  if (epoch_status[1] != 0u) return;

  // 1. publish this rank's partial
  {
    uint4 *mine = reinterpret_cast<uint4 *>(static_cast<char *>(bufs[rank]) + slot_off);
    const uint4 *src = reinterpret_cast<const uint4 *>(partial);
    for (int c = tid; c < total_chunks; c += LN_THREADS) mine[c] = src[c];
  }
  __syncthreads();
  // 2. signal every peer, 3. wait for every peer
  if (tid < world && tid != rank) {
    __threadfence_system();
    st_release_sys(flags[tid] + rank, want);
    const unsigned *f = flags[rank] + tid;
    const unsigned long long t_start = global_timer_ns();
    // flags only grow; a later epoch from a faster peer also satisfies the wait
    while ((int)(ld_acquire_sys(f) - want) < 0) {
      if (global_timer_ns() - t_start > AR_WAIT_LIMIT_NS) {
        failed = 1;
        break;
      }
      __nanosleep(100);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (failed) {
    if (tid == 0) {
      epoch_status[1] = (unsigned)DJV_ERR_TIMEOUT;
      epoch_status[0] = want;
    }
    return;
  }

  // 4. reduce in rank order, residual add, LayerNorm
  for (int row = 0; row < B; ++row) {
    const size_t off = (size_t)row * d;
    float vals[LN_MAX_CHUNKS][8];
    // All peers' pieces of two chunks are requested before the first one is used: one NVLink round trip per
    // pair of chunks instead of one per peer.
    constexpr int G = 2;
#pragma unroll
    for (int c0 = 0; c0 < LN_MAX_CHUNKS; c0 += G) {
      uint4 v[G][AR_MAX_WORLD];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int ch = (c0 + g) * LN_THREADS + tid;
#pragma unroll
        for (int p = 0; p < AR_MAX_WORLD; ++p) {
          if (ch < nchunks && p < world) {
            const char *src = static_cast<const char *>(bufs[p]) + slot_off + (off + (size_t)ch * 8) * 2;
            v[g][p] = ld_peer16(src);
          } else {
            v[g][p] = make_uint4(0, 0, 0, 0);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int c = c0 + g;
        const int ch = c * LN_THREADS + tid;
        if (ch < nchunks) {
          float f[8], t[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = 0.f;
#pragma unroll
          for (int p = 0; p < AR_MAX_WORLD; ++p) {  // rank order; absent ranks hold zeros
            unpack8(v[g][p], t);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] += t[e];
          }
          round_store8(f, nullptr);  // the all-reduced activation is an fp16 tensor
          if (residual) {
            unpack8(*reinterpret_cast<const uint4 *>(residual + off + (size_t)ch * 8), t);
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
    }
    layernorm_store(vals, nchunks, d, gamma, beta, eps, y + off, red);
  }
  if (tid == 0) epoch_status[0] = want;
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

// Set-up call: allocates three small device tables with cudaMalloc (the only allocating entry point).
extern "C" int djv_comm_create(djv_comm **out, int rank, int world, void *const *bufs,
                               void *const *flags, size_t slot_bytes, int slots) {
  DJV_REQUIRE(out && bufs && flags, "comm_create: null pointer");
  DJV_REQUIRE(world >= 1 && world <= AR_MAX_WORLD && rank >= 0 && rank < world,
              "comm_create: rank %d / world %d (max %d)", rank, world, AR_MAX_WORLD);
  DJV_REQUIRE(slots == 2, "comm_create: exactly 2 slots are used");
  DJV_REQUIRE(slot_bytes >= 16 && slot_bytes % 256 == 0, "comm_create: slot_bytes must be a multiple of 256");
  for (int r = 0; r < world; ++r)
    DJV_REQUIRE(bufs[r] && flags[r] && aligned16(bufs[r]), "comm_create: rank %d buffer/flags missing", r);
  djv_comm *c = new djv_comm();
  c->rank = rank; c->world = world; c->slots = slots; c->slot_bytes = slot_bytes;
  c->last_stream = nullptr;
  cudaError_t e = cudaMalloc(&c->bufs_dev, sizeof(void *) * AR_MAX_WORLD);
  if (e == cudaSuccess) e = cudaMalloc(&c->flags_dev, sizeof(void *) * AR_MAX_WORLD);
  if (e == cudaSuccess) e = cudaMalloc(&c->epoch_dev, 2 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemcpy(c->bufs_dev, bufs, sizeof(void *) * world, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(c->flags_dev, flags, sizeof(void *) * world, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(c->epoch_dev, 0, 2 * sizeof(unsigned));
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
  if (c->flags_dev) cudaFree(c->flags_dev);
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
  DJV_REQUIRE(c && y && partial && gamma && beta, "allreduce_add_layernorm: null pointer");
  DJV_REQUIRE(B >= 1 && d >= 8 && d % 8 == 0 && d / 8 <= LN_THREADS * LN_MAX_CHUNKS,
              "allreduce_add_layernorm: bad B=%d d=%d", B, d);
  DJV_REQUIRE((size_t)B * d * 2 <= c->slot_bytes, "allreduce_add_layernorm: %zu bytes exceed the slot (%zu)",
              (size_t)B * d * 2, c->slot_bytes);
  DJV_REQUIRE(aligned16(y) && aligned16(partial) && aligned16(gamma) && aligned16(beta) &&
                  (!r_out || aligned16(r_out)) && (!residual || aligned16(residual)),
              "allreduce_add_layernorm: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  c->last_stream = st;
  djv::launch_kernel(allreduce_add_layernorm_kernel, 1, LN_THREADS, 0, st, c->bufs_dev, c->flags_dev, c->epoch_dev, c->rank, c->world, c->slot_bytes, static_cast<__half *>(y),
      static_cast<__half *>(r_out), static_cast<const __half *>(partial),
      static_cast<const __half *>(residual), static_cast<const __half *>(gamma),
      static_cast<const __half *>(beta), B, d, eps);
  count_launch();
  return check_launch("allreduce_add_layernorm");
}
