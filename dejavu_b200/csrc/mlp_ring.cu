// Sparse MLP in ONE pass over the gathered rows, and the tensor-parallel exchange + LayerNorm in front of it:
//
//   x   = LayerNorm(sum over ranks of the attention partials + residual)      (optional prologue, exchange.cuh)
//   h_m = relu(W1[idx[m], :] . x + b1[idx[m]])   rounded to fp16
//   y   = sum_m h_m * W2t[idx[m], :] + b2         -> y, or straight into every rank's receive buffer
//
// Work split. A thread-block cluster of 8 blocks owns a contiguous range of the index list; block j of the
// cluster owns columns [j*d/8, (j+1)*d/8) of BOTH matrices. Per gathered row a block therefore streams two
// segments of d/8 halves (3 KB each at d = 12288): the dot product of row m is the sum of the 8 blocks' partial
// dots (exchanged through distributed shared memory, once per batch of rows), and the block accumulates
// h_m * W2t[idx[m], its columns] into d/8 fp32 sums held in registers (8 per thread and activation row).
// The contribution of row m to y depends on h_m only, so no grid-wide step is needed between the two products.
//
// Memory pipeline. Segments are brought into a shared-memory ring by bulk asynchronous copies (ring.cuh), up to
// 64 rows (~190 KB) in flight per block, issued by one warp, each row's pair of segments completing on its own
// mbarrier. When a cluster's share of the index list fits the ring, all of it is in flight at once and the
// cluster exchanges partial dots once; otherwise the ring is used as two halves, one being worked on while the
// copies of the other are in flight. When the caller says that the index list is complete before the launch
// (djv_set_early_weight_prefetch) and gives the row count Z, the first copies are issued BEFORE the kernel waits
// for its predecessor: the weight stream then overlaps the predecessor's tail, the NVLink trip of the exchange
// and the LayerNorm. The hint is verified: after the wait the list is read again and, should a row differ, the
// copies are started again with the right rows. For a 512-row index list everything the kernel reads is in
// flight at once.
//
// Reduction over clusters: per-cluster partial sums go to scratch, the last block to arrive for a column
// segment adds them in cluster order (deterministic) and finishes (bias, fp16, store or push).
// The same kernel runs fc1 alone (MODE 1) and fc2 alone (MODE 2).
//
// Algorithmic bytes (fp16, int32 idx): fused 2*M*d*2 + M*(2 + 4) + d*2 + 2*B*d*2.
#include <mutex>

#include "exchange.cuh"
#include "ring.cuh"

namespace djv {

constexpr int MR_THREADS = 384;
constexpr int MR_WARPS = MR_THREADS / WARP;
constexpr int MR_MAX_STAGES = 64;  // rows in flight per block
constexpr int MR_MAX_RG = 8;       // row groups of the second product
constexpr int MR_MAX_B = 4;
constexpr int MR_MAX_CLUSTERS = 40;
constexpr int MR_COUNTER_BYTES = 4096;
// shared-memory layout (bytes from the start of dynamic shared memory)
constexpr int MR_OFF_BARS = 0;      // one mbarrier per stage
constexpr int MR_OFF_PD = 512;      // [2][B][nsh] partial dots of this block (MODE 2: [B][stages] inputs h)
constexpr int MR_OFF_HS = 1536;     // [B][nsh] activations of the batch
constexpr int MR_OFF_BIAS = 2560;   // [stages] bias1 of the row in the stage
constexpr int MR_OFF_EROW = 2816;   // [stages] row index the stage's copies were started with
constexpr int MR_OFF_MISC = 3072;   // statistics, flags
constexpr int MR_OFF_X = 3840;      // [B][seg] halves, then the ring (128-byte aligned)
constexpr int MR_ISSUER = MR_WARPS - 1;  // the warp that starts the copies (the last one: with one activation row
                                         // it has no share of the exchange prologue and works beside it)
constexpr int MR_SMEM_BUDGET = 200 * 1024;

#ifdef DJV_RING_TRACE
// development build only: %globaltimer stamps of thread 0 of every block, [block][stamp]
__device__ unsigned long long g_ring_trace[512][12];
#define DJV_STAMP(i)                                                            \
  do {                                                                          \
    if (threadIdx.x == 0 && blockIdx.x < 512) {                                 \
      unsigned long long t_;                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                    \
      g_ring_trace[blockIdx.x][i] = t_;                                         \
    }                                                                           \
  } while (0)
#else
#define DJV_STAMP(i) \
  do {               \
  } while (0)
#endif

__device__ unsigned g_ring_timeouts;     // bounded waits on bulk copies that ran out (never, in a healthy run)
__device__ unsigned g_ring_bad_indices;  // index values outside [0, Z) met when the caller asked for the check

struct RingArgs {
  const __half *w1, *w2;  // (Z,N) rows of stride ldw1 / ldw2; w2 is W2 transposed
  long long ldw1, ldw2;
  const void *idx;
  int idx64;
  const __half *bias1, *bias2;
  int M, N, act;
  const __half *x;     // (B,N) input of the first product (MODE 0, 1) unless fold
  const __half *h_in;  // (B,M) input of the second product (MODE 2)
  int fold;            // x comes from the exchange
  FoldArgs f;
  __half *y;           // (B,N) (MODE 0, 2) or (B,M) (MODE 1); unused when pushing
  PushTarget push;
  float *partial;
  unsigned *counters;
  int rpc;    // rows per cluster
  int nsh;    // rows per batch
  int nbuf;   // batches in flight: 1 (all rows of the cluster fit the ring) or 2
  int early;  // start the first copies before the wait on the predecessor (needs zrows)
  int zrows;  // rows of w1 / w2 when index values are to be checked, else 0
};

__device__ __forceinline__ float apply_act_rt(int act, float v) {
  switch (act) {
    case DJV_ACT_RELU: return apply_act<DJV_ACT_RELU>(v);
    case DJV_ACT_GELU: return apply_act<DJV_ACT_GELU>(v);
    case DJV_ACT_GELU_APPROX: return apply_act<DJV_ACT_GELU_APPROX>(v);
    case DJV_ACT_SQUARED_RELU: return apply_act<DJV_ACT_SQUARED_RELU>(v);
    default: return v;
  }
}

template <int B, int MODE, int C>
__global__ void __cluster_dims__(C, 1, 1) __launch_bounds__(MR_THREADS, 1) mlp_ring_kernel(RingArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, warp = tid / WARP, lane = tid % WARP;
  const int crank = (int)cluster.block_rank();
  const int cl = blockIdx.x / C, n_cl = gridDim.x / C;
  const int seg = a.N / C, CH = seg / 8;
  const unsigned seg_bytes = (unsigned)seg * 2u;
  const unsigned stage_bytes = (MODE == 0 ? 2u : 1u) * seg_bytes;
  const int nsh = a.nsh, nbuf = a.nbuf, nstages = nsh * nbuf;

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + MR_OFF_BARS);
  float *pd = reinterpret_cast<float *>(smem + MR_OFF_PD);
  float *hs = reinterpret_cast<float *>(smem + MR_OFF_HS);
  float *bias_s = reinterpret_cast<float *>(smem + MR_OFF_BIAS);
  int *erow = reinterpret_cast<int *>(smem + MR_OFF_EROW);
  float *misc = reinterpret_cast<float *>(smem + MR_OFF_MISC);
  float *st = misc, *stf = misc + 16, *red = misc + 32;  // [4][4], [4][2], [12][4][3]
  int *flags_s = reinterpret_cast<int *>(misc + 24);     // [0] fold failed, [1] ring wait ran out, [2] last block,
                                                         // [3] phase offset of the barriers
  __half *x_s = reinterpret_cast<__half *>(smem + MR_OFF_X);
  unsigned char *ring = smem + ((MR_OFF_X + (MODE == 2 ? 0 : B * seg * 2) + 127) & ~127);

  DJV_STAMP(0);
  const int m_begin = min(a.M, cl * a.rpc), m_end = min(a.M, m_begin + a.rpc);
  const int nrows = m_end - m_begin;
  const int nbatch = (nrows + nsh - 1) / nsh;

  if (tid < nstages) mbar_init(&bars[tid], 1);
  if (tid == 0) {
    flags_s[1] = 0;
    flags_s[2] = 0;
    flags_s[3] = 0;
  }
  mbar_fence_init();
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Row index of entry m of the index list, made safe: with zrows > 0 a value outside [0, zrows) reads row 0
  // instead (counted when `count`: then it is the caller's mistake, not a list that was still being written).
  auto safe_row = [&](int m, bool count) -> long long {
    long long r = load_index(a.idx, m, a.idx64);
    if (a.zrows > 0 && (r < 0 || r >= a.zrows)) {
      if (count) atomicAdd(&g_ring_bad_indices, 1u);
      r = 0;
    }
    return r;
  };
  // warp 0: start the copies of batch bi (lane l takes rows l, l + 32 of the batch). `final_idx`: the index list is
  // known to be complete, so the per-row side data (bias1 / h) is fetched as well.
  auto issue = [&](int bi, bool final_idx, bool side) {
    const int r0 = bi * nsh, nr = min(nsh, nrows - r0), sbase = (bi % nbuf) * nsh;
    long long rr[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int s = lane + k * WARP;
      rr[k] = (s < nr) ? safe_row(m_begin + r0 + s, final_idx) : 0;
    }
    if (MODE == 2) {  // the inputs h of the rows, written before the arrival that their readers acquire
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int s = lane + k * WARP;
        if (s < nr) {
#pragma unroll
          for (int b = 0; b < B; ++b)
            pd[b * nstages + sbase + s] = __half2float(a.h_in[(size_t)b * a.M + m_begin + r0 + s]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int s = lane + k * WARP;
      if (s < nr) {
        const long long r = rr[k];
        const int stg = sbase + s;
        uint64_t *bar = &bars[stg];
        unsigned char *dst = ring + (size_t)stg * stage_bytes;
        mbar_arrive_expect_tx(bar, stage_bytes);
        if (MODE != 2) {
          bulk_load(dst, a.w1 + r * a.ldw1 + (size_t)crank * seg, seg_bytes, bar);
          dst += seg_bytes;
        }
        if (MODE != 1) bulk_load(dst, a.w2 + r * a.ldw2 + (size_t)crank * seg, seg_bytes, bar);
        erow[stg] = (int)r;
      }
    }
    if (MODE != 2 && side) {  // bias1 of the rows, once the copies are on their way
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int s = lane + k * WARP;
        if (s < nr) bias_s[sbase + s] = a.bias1 ? __half2float(a.bias1[rr[k]]) : 0.f;
      }
    }
  };
  // The caller's hint that the index list is complete lets the weight stream start before the wait on the
  // predecessor. It is only a hint: after the wait the list is read again, and if any row differs (the list was
  // still being written) every copy is started again with the right rows, one barrier phase later.
  const bool early = a.early != 0 && a.zrows > 0 && MODE != 2;
  if (early && warp == MR_ISSUER) {
    for (int bi = 0; bi < nbuf && bi < nbatch; ++bi) issue(bi, false, false);
  }
  FoldRegs<B> fr;
  FoldCtx fctx{};
  const int c_lo = crank * CH, c_hi = c_lo + CH;
  if (MODE != 2 && a.fold) {
    fold_fetch_affine<MR_THREADS, B>(fr, a.f, c_lo, c_hi, 0, B);
    fctx = fold_begin(a.f);
  }
  DJV_STAMP(1);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  DJV_STAMP(2);
  // The issuer re-reads, now that the list is certainly complete, the rows its early copies were started with.
  // The loads are issued here and compared after the prologue below, so that they overlap it.
  long long r_true[2][2];
  if (warp == MR_ISSUER) {
    if (early) {
      for (int bi = 0; bi < nbuf && bi < 2 && bi < nbatch; ++bi) {
        const int r0 = bi * nsh, nr = min(nsh, nrows - r0);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int s = lane + k * WARP;
          // (raw value: it is not looked at before the comparison below, so the load overlaps the prologue)
          r_true[bi][k] = (s < nr) ? load_index(a.idx, m_begin + r0 + s, a.idx64) : 0;
        }
      }
    } else {
      for (int bi = 0; bi < nbuf && bi < nbatch; ++bi) issue(bi, true, false);
    }
  }

  // ---- this block's columns of the input rows ------------------------------------------------
  bool input_ok = true;
  if (MODE != 2) {
    if (a.fold) {
      input_ok = exchange_fold<MR_THREADS, B>(a.f, fctx, cluster, C, c_lo, c_hi, 0, B, cl == 0, x_s, crank,
                                              cl == 0 ? C : 0, fr, red, st, stf, &flags_s[0]);
    } else {
      for (int item = tid; item < B * CH; item += MR_THREADS) {
        const int b = item / CH, c = item % CH;
        reinterpret_cast<uint4 *>(x_s)[item] = ld_cached16(a.x + (size_t)b * a.N + (size_t)(c_lo + c) * 8);
      }
    }
  }
  if (early && warp == MR_ISSUER) {
    bool differs = false;
    for (int bi = 0; bi < nbuf && bi < 2 && bi < nbatch; ++bi) {
      const int r0 = bi * nsh, nr = min(nsh, nrows - r0), sbase = (bi % nbuf) * nsh;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int s = lane + k * WARP;
        if (s < nr) differs = differs || r_true[bi][k] != (long long)erow[sbase + s];
      }
    }
    if (__any_sync(0xffffffffu, differs)) {  // the list was still being written: start over, one phase later
      bool landed = true;
      for (int s = lane; s < min(nstages, nrows); s += WARP) landed = mbar_wait(&bars[s], 0) && landed;
      if (!landed) flags_s[1] = 1;
      __syncwarp();
      fence_proxy_async_smem();
      for (int bi = 0; bi < nbuf && bi < nbatch; ++bi) issue(bi, true, false);
      if (lane == 0) flags_s[3] = 1;
    }
  }
  __syncthreads();
  DJV_STAMP(3);
  const unsigned par_base = (unsigned)flags_s[3];
  if (MODE != 2 && warp == MR_ISSUER) {
    // bias1 of the first rows, while the other warps start on the first product (read after the cluster barrier)
    for (int bi = 0; bi < nbuf && bi < 2 && bi < nbatch; ++bi) {
      const int r0 = bi * nsh, nr = min(nsh, nrows - r0), sbase = (bi % nbuf) * nsh;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int s = lane + k * WARP;
        if (s < nr) bias_s[sbase + s] = a.bias1 ? __half2float(a.bias1[erow[sbase + s]]) : 0.f;
      }
    }
  }

  // ---- main loop over batches of rows ----------------------------------------------------------
  const int RG = min(MR_THREADS / CH, MR_MAX_RG);
  const int rg = tid / CH, cc = tid % CH;  // second product: this thread's row group and 16-byte column chunk
  const bool colthread = rg < RG;
  float acc[B][8];
#pragma unroll
  for (int b = 0; b < B; ++b)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[b][e] = 0.f;
  bool ring_ok = true;
  const uint4 *xs4 = reinterpret_cast<const uint4 *>(x_s);

  for (int bi = 0; bi < nbatch; ++bi) {
    const int r0 = bi * nsh, nr = min(nsh, nrows - r0), sbase = (bi % nbuf) * nsh;
    const unsigned par = ((unsigned)(bi / nbuf) + par_base) & 1u;
    float *pdb = pd + (size_t)(bi & 1) * B * nsh;
    if (MODE != 2) {
      // first product: a warp per row, partial dot over this block's columns (two independent sums per lane)
      for (int s = warp; s < nr; s += MR_WARPS) {
        ring_ok = ring_ok && mbar_wait(&bars[sbase + s], par);
        const uint4 *w = reinterpret_cast<const uint4 *>(ring + (size_t)(sbase + s) * stage_bytes);
        float p0[B], p1[B];
#pragma unroll
        for (int b = 0; b < B; ++b) p0[b] = p1[b] = 0.f;
        int c = lane;
        for (; c + WARP < CH; c += 2 * WARP) {
          const uint4 wa = w[c], wb = w[c + WARP];
#pragma unroll
          for (int b = 0; b < B; ++b) {
            p0[b] = dot8(wa, xs4[b * CH + c], p0[b]);
            p1[b] = dot8(wb, xs4[b * CH + c + WARP], p1[b]);
          }
        }
        if (c < CH) {
          const uint4 wa = w[c];
#pragma unroll
          for (int b = 0; b < B; ++b) p0[b] = dot8(wa, xs4[b * CH + c], p0[b]);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) p0[b] = warp_sum(p0[b] + p1[b]);
        if (lane == 0) {
#pragma unroll
          for (int b = 0; b < B; ++b) pdb[b * nsh + s] = p0[b];
        }
      }
      if (bi == 0) DJV_STAMP(4);
      cluster.sync();  // every block's partial dots of this batch are in its shared memory
      if (bi == 0) DJV_STAMP(5);
      if (MODE == 1 && warp == MR_ISSUER && bi + nbuf < nbatch) {  // fc1 alone: the batch's stages are free already
        fence_proxy_async_smem();
        issue(bi + nbuf, true, true);
      }
      // activations of the batch (every block of the cluster computes the same values, in the same order)
      for (int item = tid; item < nr * B; item += MR_THREADS) {
        const int s = item / B, b = item % B;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < C; ++j) sum += cluster.map_shared_rank(pdb, j)[b * nsh + s];
        sum += bias_s[sbase + s];
        const __half hv = __float2half_rn(apply_act_rt(a.act, sum));  // h is an fp16 tensor between the products
        if (MODE == 1 && crank == 0) a.y[(size_t)b * a.M + m_begin + r0 + s] = hv;
        hs[b * nsh + s] = __half2float(hv);
      }
      if (MODE == 1) continue;  // (pd is double-buffered: the next cluster barrier orders its reuse)
      __syncthreads();
      if (bi == 0) DJV_STAMP(6);
    }
    // second product: thread (rg, cc) adds rows rg, rg + RG, ... of the batch into its 8 columns, four rows'
    // loads at a time. MODE 0: every row of the batch was seen complete by the warp that took its first product,
    // before the block-wide barriers above; MODE 2: each thread waits for the row's copy itself.
    if (colthread) {
      auto w2_chunk = [&](int s) -> uint4 {
        return *reinterpret_cast<const uint4 *>(ring + (size_t)(sbase + s) * stage_bytes +
                                                (MODE == 0 ? seg_bytes : 0u) + (size_t)cc * 16);
      };
      auto add_row = [&](int s, const uint4 &wv) {
        const float2 w0 = h2f(wv.x), w1 = h2f(wv.y), w2 = h2f(wv.z), w3 = h2f(wv.w);
#pragma unroll
        for (int b = 0; b < B; ++b) {
          const float hb = (MODE == 2) ? pd[b * nstages + sbase + s] : hs[b * nsh + s];
          acc[b][0] = fmaf(hb, w0.x, acc[b][0]);
          acc[b][1] = fmaf(hb, w0.y, acc[b][1]);
          acc[b][2] = fmaf(hb, w1.x, acc[b][2]);
          acc[b][3] = fmaf(hb, w1.y, acc[b][3]);
          acc[b][4] = fmaf(hb, w2.x, acc[b][4]);
          acc[b][5] = fmaf(hb, w2.y, acc[b][5]);
          acc[b][6] = fmaf(hb, w3.x, acc[b][6]);
          acc[b][7] = fmaf(hb, w3.y, acc[b][7]);
        }
      };
      int s = rg;
      for (; s + 3 * RG < nr; s += 4 * RG) {
        if (MODE == 2) {
#pragma unroll
          for (int u = 0; u < 4; ++u) ring_ok = ring_ok && mbar_wait(&bars[sbase + s + u * RG], par);
        }
        uint4 wv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) wv[u] = w2_chunk(s + u * RG);
#pragma unroll
        for (int u = 0; u < 4; ++u) add_row(s + u * RG, wv[u]);
      }
      for (; s < nr; s += RG) {
        if (MODE == 2) ring_ok = ring_ok && mbar_wait(&bars[sbase + s], par);
        add_row(s, w2_chunk(s));
      }
    }
    if (bi + nbuf < nbatch) {
      __syncthreads();  // the batch's stages (and hs) are free
      if (warp == MR_ISSUER) {
        fence_proxy_async_smem();
        issue(bi + nbuf, true, true);
      }
    }
  }
  if (!ring_ok) flags_s[1] = 1;
  DJV_STAMP(7);
  cluster.sync();  // no block leaves (or reuses the ring) while a peer may still read its shared memory
  if (flags_s[1] != 0 && tid == 0) atomicAdd(&g_ring_timeouts, 1u);
  const bool ok = input_ok && flags_s[1] == 0;
  if (MODE == 1) return;

  // ---- row groups -> block -> clusters -> result ---------------------------------------------------
  float *redv = reinterpret_cast<float *>(ring);  // [RG][B][seg]; every copy into the ring has completed
  if (colthread) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float4 *dst = reinterpret_cast<float4 *>(redv + ((size_t)rg * B + b) * seg + (size_t)cc * 8);
      dst[0] = make_float4(acc[b][0], acc[b][1], acc[b][2], acc[b][3]);
      dst[1] = make_float4(acc[b][4], acc[b][5], acc[b][6], acc[b][7]);
    }
  }
  __syncthreads();
  const int gcol0 = crank * seg;
  size_t piece_off = 0;
  if (a.push.bufs != nullptr) piece_off = push_piece_offset(a.push);
  // bias2 of the chunk this thread finishes first, requested before the partial sums are waited for
  const uint4 bias2_pre = (a.bias2 != nullptr && tid < B * CH) ? ld_cached16(a.bias2 + gcol0 + (tid % CH) * 8)
                                                                : make_uint4(0, 0, 0, 0);
  auto emit = [&](int b, int c, float (&v)[8]) {
    const int gcol = gcol0 + c * 8;
    if (a.bias2 != nullptr) {
      float t8[8];
      unpack8f((b * CH + c == tid) ? bias2_pre : ld_cached16(a.bias2 + gcol), t8);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += t8[e];
    }
    const uint4 packed = round8(v);
    if (!ok) return;
    if (a.push.bufs != nullptr)
      push16(a.push, piece_off, (size_t)b * a.N + gcol, packed);
    else
      *reinterpret_cast<uint4 *>(a.y + (size_t)b * a.N + gcol) = packed;
  };
  for (int item = tid; item < B * CH; item += MR_THREADS) {
    const int b = item / CH, c = item % CH;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    for (int g = 0; g < RG; ++g) {
      const float4 *src = reinterpret_cast<const float4 *>(redv + ((size_t)g * B + b) * seg + (size_t)c * 8);
      const float4 lo = src[0], hi = src[1];
      v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
      v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
    }
    if (n_cl == 1) {
      emit(b, c, v);
    } else {
      float4 *dst = reinterpret_cast<float4 *>(a.partial + ((size_t)cl * B + b) * a.N + gcol0 + c * 8);
      __stcg(dst, make_float4(v[0], v[1], v[2], v[3]));
      __stcg(dst + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
  }
  if (n_cl == 1) return;
  DJV_STAMP(8);
  // several clusters: the last block to arrive for this column segment adds their sums in cluster order
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned ticket = atomicAdd(&a.counters[crank], 1u);
    flags_s[2] = (ticket == (unsigned)n_cl - 1u) ? 1 : 0;
  }
  __syncthreads();
  DJV_STAMP(9);
  if (flags_s[2] == 0) return;
  __threadfence();
  // The n_cl partial sums of a chunk are split into KS contiguous slices of clusters, one thread per (chunk,
  // slice); a thread requests up to 8 partials at a time before it adds them, in cluster order; the slices are
  // then added in slice order. The order is fixed by (n_cl, KS): results are deterministic.
  const int items = B * CH;
  int KS = 1;
  while (KS < 4 && items * KS * 2 <= MR_THREADS && KS * 2 <= n_cl) KS *= 2;
  const int per = (n_cl + KS - 1) / KS;
  float *slice = redv;  // [KS][items][8], reuses the row-group buffer (all reads of it are done)
  __syncthreads();
  for (int w = tid; w < items * KS; w += MR_THREADS) {
    const int item = w % items, ks = w / items;
    const int b = item / CH, c = item % CH;
    const int k_lo = ks * per, k_hi = min(n_cl, k_lo + per);
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    for (int k0 = k_lo; k0 < k_hi; k0 += 8) {
      float4 lo[8], hi[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k0 + u < k_hi) {
          const float4 *src =
              reinterpret_cast<const float4 *>(a.partial + ((size_t)(k0 + u) * B + b) * a.N + gcol0 + c * 8);
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
    if (KS == 1) {
      emit(b, c, v);
    } else {
      float4 *dst = reinterpret_cast<float4 *>(slice + ((size_t)ks * items + item) * 8);
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  if (KS > 1) {
    __syncthreads();
    for (int item = tid; item < items; item += MR_THREADS) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
      for (int ks = 0; ks < KS; ++ks) {
        const float4 *src = reinterpret_cast<const float4 *>(slice + ((size_t)ks * items + item) * 8);
        const float4 lo = src[0], hi = src[1];
        v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
        v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
      }
      emit(item / CH, item % CH, v);
    }
  }
  if (tid == 0) a.counters[crank] = 0;  // ready for the next launch
  DJV_STAMP(10);
}

}  // namespace djv

using namespace djv;

namespace {

inline size_t ring_fixed_bytes(int B, int N, int mode, int C) {
  const int seg = N / C;
  return (size_t)((MR_OFF_X + (mode == 2 ? 0 : B * seg * 2) + 127) & ~127);
}

inline size_t ring_smem_bytes(int B, int N, int mode, int C, int nstages) {
  const int seg = N / C, CH = seg / 8;
  const size_t stage = (size_t)(mode == 0 ? 2 : 1) * seg * 2;
  int RG = MR_THREADS / CH;
  if (RG > MR_MAX_RG) RG = MR_MAX_RG;
  size_t ring = (size_t)nstages * stage;
  const size_t redv = mode == 1 ? 0 : (size_t)RG * B * seg * sizeof(float);
  if (ring < redv) ring = redv;
  return ring_fixed_bytes(B, N, mode, C) + ring;
}

template <int B, int MODE, int C>
int ring_max_clusters(size_t smem) {
  // clusters of this kernel the device holds at once, per shared-memory size (a handful of distinct sizes)
  static std::mutex mu;
  static size_t keys[16];
  static int vals[16];
  static int n = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n; ++i)
    if (keys[i] == smem) return vals[i];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C, 1, 1);
  cfg.blockDim = dim3(MR_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int got = 0;
  if (cudaOccupancyMaxActiveClusters(&got, mlp_ring_kernel<B, MODE, C>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    got = 0;
  }
  if (got <= 0) got = sm_count() / C * 7 / 8;  // fall-back: what the cluster granularity of a GPC loses
  if (n < 16) {
    keys[n] = smem;
    vals[n] = got;
    ++n;
  }
  return got;
}

template <int B, int MODE, int C>
int ring_prepare() {
  static int rc = [] {
    cudaError_t e = cudaFuncSetAttribute(mlp_ring_kernel<B, MODE, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         MR_SMEM_BUDGET + 8192);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return 1;
    }
    return 0;
  }();
  return rc;
}

template <int B, int MODE, int C>
int ring_launch(RingArgs a, cudaStream_t st) {
  if (ring_prepare<B, MODE, C>() != 0) {
    set_error("mlp_ring: cannot raise the kernel's shared-memory limit");
    return DJV_ERR_CUDA;
  }
  const int seg = a.N / C;
  const size_t stage = (size_t)(MODE == 0 ? 2 : 1) * seg * 2;
  const size_t fixed = ring_fixed_bytes(B, a.N, MODE, C);
  int stages_max = (int)((MR_SMEM_BUDGET - fixed) / stage);
  if (stages_max > MR_MAX_STAGES) stages_max = MR_MAX_STAGES;
  if (stages_max < 2) {
    set_error("mlp_ring: N=%d rows do not fit the shared-memory ring", a.N);
    return DJV_ERR_UNSUPPORTED;
  }
  static const int k_cl = env_int("DJV_RING_CLUSTERS", 0);  // development knob
  int maxcl = k_cl > 0 ? k_cl : ring_max_clusters<B, MODE, C>(ring_smem_bytes(B, a.N, MODE, C, stages_max));
  if (maxcl > MR_MAX_CLUSTERS) maxcl = MR_MAX_CLUSTERS;
  if (maxcl < 1) maxcl = 1;
  // at least 4 rows per cluster; then even shares
  int n_cl = ceil_div(a.M, 4);
  if (n_cl > maxcl) n_cl = maxcl;
  const int rpc = ceil_div(a.M, n_cl);
  n_cl = ceil_div(a.M, rpc);
  // all rows of a cluster in flight at once when the ring holds them (one batch, one exchange of partial dots);
  // otherwise two half-rings: one batch is worked on while the copies of the next are in flight
  int nsh, nbuf;
  if (rpc <= stages_max) {
    nsh = rpc;
    nbuf = 1;
  } else {
    nsh = stages_max / 2;
    nbuf = 2;
  }
  a.rpc = rpc;
  a.nsh = nsh;
  a.nbuf = nbuf;
  const size_t smem = ring_smem_bytes(B, a.N, MODE, C, nsh * nbuf);
  static const int k_dbg = env_int("DJV_RING_DEBUG", 0);  // development knob: print the plan
  if (k_dbg)
    fprintf(stderr, "mlp_ring<B=%d,MODE=%d,C=%d>: M=%d N=%d clusters=%d (device holds %d) rows/cluster=%d rows/batch=%d "
                    "batches in flight=%d smem=%zu early=%d fold=%d\n", B, MODE, C, a.M, a.N, n_cl, maxcl, rpc, nsh,
            nbuf, smem, a.early, a.fold);
  djv::launch_kernel(mlp_ring_kernel<B, MODE, C>, dim3(n_cl * C), dim3(MR_THREADS), smem, st, a);
  count_launch();
  return DJV_OK;
}

// blocks per cluster = column segments: 8 unless the development knob DJV_RING_C says 4
static int ring_cluster_size(int N) {
  static const int k_c = env_int("DJV_RING_C", 8);
  int c = (k_c == 4) ? 4 : 8;
  if (c == 4 && (N % 32 != 0 || N / 32 > MR_THREADS)) c = 8;
  return c;
}

template <int MODE>
int ring_dispatch(int B, const RingArgs &a, cudaStream_t st) {
  const bool c4 = ring_cluster_size(a.N) == 4;
  switch (B) {
    case 1: return c4 ? ring_launch<1, MODE, 4>(a, st) : ring_launch<1, MODE, 8>(a, st);
    case 2: return c4 ? ring_launch<2, MODE, 4>(a, st) : ring_launch<2, MODE, 8>(a, st);
    case 3: return c4 ? ring_launch<3, MODE, 4>(a, st) : ring_launch<3, MODE, 8>(a, st);
    case 4: return c4 ? ring_launch<4, MODE, 4>(a, st) : ring_launch<4, MODE, 8>(a, st);
  }
  set_error("mlp_ring: batch %d outside [1,%d]", B, MR_MAX_B);
  return DJV_ERR_INVALID;
}

int ring_check(const char *op, int B, int N, int M, long long ld1, long long ld2, const void *w1, const void *w2,
               void *scratch, size_t scratch_bytes) {
  DJV_REQUIRE(B >= 1 && B <= MR_MAX_B, "%s: batch %d outside [1,%d]", op, B, MR_MAX_B);
  DJV_REQUIRE(N >= 64 && N % (8 * 8) == 0 && N / (8 * 8) <= MR_THREADS,
              "%s: N=%d must be a multiple of %d and at most %d", op, N, 8 * 8, 8 * 8 * MR_THREADS);
  DJV_REQUIRE(M >= 1, "%s: needs at least one row", op);
  DJV_REQUIRE((!w1 || (ld1 >= N && ld1 % 8 == 0 && aligned16(w1))) && (!w2 || (ld2 >= N && ld2 % 8 == 0 && aligned16(w2))),
              "%s: weights must be 16-byte aligned with row strides >= N that are multiples of 8", op);
  const size_t need = djv_mlp_sparse_fused_scratch_bytes(B, N, M);
  if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
    set_error("%s: scratch needs %zu bytes, 256-byte aligned (got %zu)", op, need, scratch_bytes);
    return DJV_ERR_SCRATCH;
  }
  return DJV_OK;
}

void ring_scratch(RingArgs &a, void *scratch) {
  a.counters = reinterpret_cast<unsigned *>(scratch);
  a.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + MR_COUNTER_BYTES);
}

}  // namespace

extern "C" int djv_mlp_sparse_fused_supported(int B, int N, int M) {
  return B >= 1 && B <= MR_MAX_B && N >= 64 && N % (8 * 8) == 0 && N / (8 * 8) <= MR_THREADS && M >= 1;
}

// 1 when the plan keeps every row of a cluster in flight at once (one exchange of partial dots per cluster): the
// regime of short index lists the one-pass kernel is made for. Needs a CUDA device (occupancy query).
extern "C" int djv_mlp_sparse_fused_single_batch(int B, int N, int M) {
  if (!djv_mlp_sparse_fused_supported(B, N, M)) return 0;
  const int C = 8;
  const size_t stage = (size_t)2 * (N / C) * 2;
  const size_t fixed = ring_fixed_bytes(B, N, 0, C);
  int stages_max = (int)((MR_SMEM_BUDGET - fixed) / stage);
  if (stages_max > MR_MAX_STAGES) stages_max = MR_MAX_STAGES;
  if (stages_max < 2) return 0;
  int maxcl = sm_count() / C * 7 / 8;  // what the cluster granularity of a GPC leaves (15 on a 148-SM part)
  if (maxcl > MR_MAX_CLUSTERS) maxcl = MR_MAX_CLUSTERS;
  if (maxcl < 1) maxcl = 1;
  int n_cl = ceil_div(M, 4);
  if (n_cl > maxcl) n_cl = maxcl;
  return ceil_div(M, n_cl) <= stages_max ? 1 : 0;
}

extern "C" size_t djv_mlp_sparse_fused_scratch_bytes(int B, int N, int M) {
  if (B < 1 || N < 8 || M < 0) return 0;
  return MR_COUNTER_BYTES + (size_t)MR_MAX_CLUSTERS * B * N * sizeof(float);
}

extern "C" unsigned djv_mlp_ring_timeouts(void) {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ring_timeouts, sizeof(v)) != cudaSuccess) {
    cudaGetLastError();
    return ~0u;
  }
  return v;
}

#ifdef DJV_RING_TRACE
extern "C" int djv_mlp_ring_trace(unsigned long long *out) {
  return cudaMemcpyFromSymbol(out, g_ring_trace, sizeof(g_ring_trace)) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" unsigned djv_mlp_ring_bad_indices(void) {
  unsigned v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ring_bad_indices, sizeof(v)) != cudaSuccess) {
    cudaGetLastError();
    return ~0u;
  }
  return v;
}

extern "C" int djv_mlp_sparse_fused(void *y, const void *w1, const void *w2t, const void *x, const void *idx,
                                    const void *bias1, const void *bias2, int B, int N, int M, int Z, long long ldw1,
                                    long long ldw2t, int idx_is_64, void *scratch, size_t scratch_bytes,
                                    void *stream) {
  DJV_REQUIRE(y && w1 && w2t && x && idx, "mlp_sparse_fused: null pointer");
  int rc = ring_check("mlp_sparse_fused", B, N, M, ldw1, ldw2t, w1, w2t, scratch, scratch_bytes);
  if (rc) return rc;
  DJV_REQUIRE(aligned16(x) && aligned16(y) && (!bias2 || aligned16(bias2)),
              "mlp_sparse_fused: x, y and bias2 must be 16-byte aligned");
  RingArgs a{};
  a.w1 = static_cast<const __half *>(w1);
  a.w2 = static_cast<const __half *>(w2t);
  a.ldw1 = ldw1; a.ldw2 = ldw2t;
  a.idx = idx; a.idx64 = idx_is_64;
  a.bias1 = static_cast<const __half *>(bias1);
  a.bias2 = static_cast<const __half *>(bias2);
  a.M = M; a.N = N; a.act = DJV_ACT_RELU;
  a.zrows = Z > 0 ? Z : 0;
  a.x = static_cast<const __half *>(x);
  a.y = static_cast<__half *>(y);
  a.early = early_prefetch() ? 1 : 0;
  ring_scratch(a, scratch);
  rc = ring_dispatch<0>(B, a, static_cast<cudaStream_t>(stream));
  if (rc) return rc;
  return check_launch("mlp_sparse_fused");
}

extern "C" int djv_mlp_sparse_fused_exchange(djv_comm *comm, int seq_in, int flags, int seq_out, void *y,
                                             void *r_out, const void *residual, const void *gamma,
                                             const void *beta, float eps, const void *w1, const void *w2t,
                                             const void *idx, const void *bias1, const void *bias2, int B, int N,
                                             int M, int Z, long long ldw1, long long ldw2t, int idx_is_64,
                                             void *scratch, size_t scratch_bytes, void *stream) {
  DJV_REQUIRE(comm && w1 && w2t && idx && gamma && beta, "mlp_sparse_fused_exchange: null pointer");
  DJV_REQUIRE(seq_in >= 0 && (seq_out >= 0 || y != nullptr),
              "mlp_sparse_fused_exchange: needs an input exchange and an output (exchange number or y)");
  int rc = ring_check("mlp_sparse_fused_exchange", B, N, M, ldw1, ldw2t, w1, w2t, scratch, scratch_bytes);
  if (rc) return rc;
  DJV_REQUIRE((size_t)B * N * 2 <= comm->slot_bytes, "mlp_sparse_fused_exchange: %zu bytes exceed the slot (%zu)",
              (size_t)B * N * 2, comm->slot_bytes);
  DJV_REQUIRE((!y || aligned16(y)) && (!r_out || aligned16(r_out)) && (!residual || aligned16(residual)) &&
                  aligned16(gamma) && aligned16(beta) && (!bias2 || aligned16(bias2)),
              "mlp_sparse_fused_exchange: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  comm->last_stream = st;
  RingArgs a{};
  a.w1 = static_cast<const __half *>(w1);
  a.w2 = static_cast<const __half *>(w2t);
  a.ldw1 = ldw1; a.ldw2 = ldw2t;
  a.idx = idx; a.idx64 = idx_is_64;
  a.bias1 = static_cast<const __half *>(bias1);
  a.bias2 = static_cast<const __half *>(bias2);
  a.M = M; a.N = N; a.act = DJV_ACT_RELU;
  a.zrows = Z > 0 ? Z : 0;
  a.fold = 1;
  a.f = fold_args(comm, seq_in);
  a.f.residual = static_cast<const __half *>(residual);
  a.f.r_out = static_cast<__half *>(r_out);
  a.f.gamma = static_cast<const __half *>(gamma);
  a.f.beta = static_cast<const __half *>(beta);
  a.f.eps = eps;
  a.f.refill = (flags & DJV_EXCHANGE_REFILL) ? 1 : 0;
  a.f.B = B;
  a.f.d = N;
  a.y = static_cast<__half *>(y);
  if (seq_out >= 0) a.push = push_target(comm, seq_out);
  a.early = early_prefetch() ? 1 : 0;
  ring_scratch(a, scratch);
  rc = ring_dispatch<0>(B, a, st);
  if (rc) return rc;
  return check_launch("mlp_sparse_fused_exchange");
}

// fc1 / fc2 alone on the same pipeline (used by djv_gather_gemv / djv_gather_transposed_gemv for short index
// lists, where bytes in flight matter most)
namespace djv {
int ring_fc1(__half *y, const __half *w, const __half *x, const void *idx, const __half *bias, int B, int N, int M,
             long long ldw, int idx64, int act, cudaStream_t st) {
  RingArgs a{};
  a.w1 = w; a.ldw1 = ldw; a.idx = idx; a.idx64 = idx64; a.bias1 = bias;
  a.M = M; a.N = N; a.act = act; a.x = x; a.y = y;
  a.early = (idx == nullptr) ? 1 : 0;  // without the row count the index values cannot be double-checked
  a.zrows = (idx == nullptr) ? M : 0;
  return ring_dispatch<1>(B, a, st);
}
int ring_fc2(__half *y, const __half *w, const __half *h, const void *idx, const __half *bias, int B, int N, int M,
             long long ldw, int idx64, void *scratch, cudaStream_t st, const PushTarget &push) {
  RingArgs a{};
  a.w2 = w; a.ldw2 = ldw; a.idx = idx; a.idx64 = idx64; a.bias2 = bias;
  a.M = M; a.N = N; a.h_in = h; a.y = y; a.push = push;
  ring_scratch(a, scratch);
  return ring_dispatch<2>(B, a, st);
}
}  // namespace djv
