// Tensor-parallel one-shot all-reduce fused with the residual add and LayerNorm that follow it, as a kernel
// of its own (the fused sparse-MLP kernel runs the same receiving code in its prologue, see exchange.cuh), and
// the set-up / tear-down of the exchange.
//
// One thread-block cluster of 8 blocks per row: each block owns an eighth of the row's 16-byte chunks, one
// chunk per thread for hidden sizes up to 16384, so all pieces of the whole row are requested in one round of
// loads; the LayerNorm statistics are merged over the cluster through distributed shared memory.
#include "exchange.cuh"

namespace djv {

constexpr int EX_THREADS = 256;
constexpr int EX_CLUSTER = 8;

__global__ void fill_sentinel_kernel(uint4 *p, size_t n16) {
  const uint4 s = make_uint4(AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2, AR_SENTINEL2);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
    p[i] = s;
}

// ctl[0] += n: the exchanges of the step that just ended. Launched once per step, after every kernel of the
// step that reads ctl[0] (all streams joined), so the value is stable while a step runs.
__global__ void comm_end_step_kernel(unsigned *ctl, unsigned n) {
  pdl_prologue();
  if (threadIdx.x == 0) ctl[0] += n;
}

template <int ITEMS, int CL, int THREADS>
__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(THREADS)
exchange_layernorm_kernel(FoldArgs a) {
  __shared__ float red[THREADS / WARP * 3];
  __shared__ float st[4], stf[2];
  __shared__ int failed_s;
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int row = blockIdx.y;
  const int nchunks = a.d / 8;
  const int per = (nchunks + CL - 1) / CL;
  const int c_lo = min(nchunks, crank * per), c_hi = min(nchunks, c_lo + per);
  // the affine weights are fetched while the predecessor kernel may still be running
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  FoldRegs<ITEMS> fr;
  fold_fetch_affine<THREADS, ITEMS>(fr, a, c_lo, c_hi, row, 1);
  const FoldCtx ctx = fold_begin(a);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  exchange_fold<THREADS, ITEMS>(a, ctx, cluster, CL, c_lo, c_hi, row, 1, true, nullptr, row * CL + crank,
                                (int)gridDim.y * CL, fr, red, st, stf, &failed_s);
  cluster.sync();  // no block leaves while a peer may still read its statistics
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
  c->bufs_dev = nullptr;
  c->ctl_dev = nullptr;
  cudaError_t e = cudaMalloc(&c->bufs_dev, sizeof(void *) * AR_MAX_WORLD);
  if (e == cudaSuccess) e = cudaMalloc(&c->ctl_dev, AR_CTL_WORDS * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemcpy(c->bufs_dev, bufs, sizeof(void *) * world, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(c->ctl_dev, 0, AR_CTL_WORDS * sizeof(unsigned));
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
  if (c->ctl_dev) cudaFree(c->ctl_dev);
  delete c;
  return DJV_OK;
}

extern "C" int djv_comm_status(djv_comm *c) {
  DJV_REQUIRE(c, "comm_status: null comm");
  unsigned es[2] = {0, 0};
  cudaError_t e = cudaStreamSynchronize(c->last_stream);
  if (e == cudaSuccess) e = cudaMemcpy(es, c->ctl_dev, sizeof(es), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_error("comm_status: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  if ((int)es[1] != 0) set_error("exchange: a peer did not arrive within the wait limit (after %u exchanges of earlier steps)", es[0]);
  return (int)es[1];
}

extern "C" int djv_comm_end_step(djv_comm *c, int n_exchanges, void *stream) {
  DJV_REQUIRE(c && n_exchanges >= 0, "comm_end_step: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  c->last_stream = st;
  if (n_exchanges == 0) return DJV_OK;
  djv::launch_kernel(comm_end_step_kernel, 1, 32, 0, st, c->ctl_dev, (unsigned)n_exchanges);
  count_launch();
  return check_launch("comm_end_step");
}

extern "C" int djv_allreduce_add_layernorm(djv_comm *c, int seq, int flags, void *y, void *r_out,
                                           const void *partial, const void *residual, const void *gamma,
                                           const void *beta, int B, int d, float eps, void *stream) {
  DJV_REQUIRE(c != nullptr, "allreduce_add_layernorm: null comm");
  DJV_REQUIRE((gamma == nullptr) == (beta == nullptr), "allreduce_add_layernorm: gamma and beta go together");
  DJV_REQUIRE(y != nullptr || r_out != nullptr, "allreduce_add_layernorm: no output pointer");
  DJV_REQUIRE(seq >= 0, "allreduce_add_layernorm: negative exchange number %d", seq);
  DJV_REQUIRE(B >= 1 && B <= DJV_MAX_BATCH && d >= 8 && d % 8 == 0 && d / 8 <= EX_CLUSTER * EX_THREADS * 2,
              "allreduce_add_layernorm: bad B=%d d=%d", B, d);
  DJV_REQUIRE((size_t)B * d * 2 <= c->slot_bytes, "allreduce_add_layernorm: %zu bytes exceed the slot (%zu)",
              (size_t)B * d * 2, c->slot_bytes);
  DJV_REQUIRE((!y || aligned16(y)) && (!partial || aligned16(partial)) && (!gamma || aligned16(gamma)) &&
                  (!beta || aligned16(beta)) && (!r_out || aligned16(r_out)) && (!residual || aligned16(residual)),
              "allreduce_add_layernorm: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  c->last_stream = st;
  FoldArgs a = fold_args(c, seq);
  a.partial = static_cast<const __half *>(partial);
  a.residual = static_cast<const __half *>(residual);
  a.r_out = static_cast<__half *>(r_out);
  a.gamma = static_cast<const __half *>(gamma);
  a.beta = static_cast<const __half *>(beta);
  a.eps = eps;
  a.y = static_cast<__half *>(y);
  a.refill = (flags & DJV_EXCHANGE_REFILL) ? 1 : 0;
  a.B = B;
  a.d = d;
  // (clusters of 4 blocks x 512 threads and a single block of 1024 threads were measured slower: 4.6 and 11 us
  // against 4.2 us for one rank at d = 9216)
  const dim3 grid(EX_CLUSTER, B);
  if (d / 8 <= EX_CLUSTER * EX_THREADS)
    djv::launch_kernel(exchange_layernorm_kernel<1, EX_CLUSTER, EX_THREADS>, grid, EX_THREADS, 0, st, a);
  else
    djv::launch_kernel(exchange_layernorm_kernel<2, EX_CLUSTER, EX_THREADS>, grid, EX_THREADS, 0, st, a);
  count_launch();
  return check_launch("allreduce_add_layernorm");
}
