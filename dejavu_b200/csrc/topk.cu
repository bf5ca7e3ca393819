// Top-K index selection over one score vector, keys held in shared memory: one block for short vectors (and for
// head lists, whose selection also opens the attention layer's decode step), a cluster of 8 blocks for long ones.
//
// Radix select (8 bits per pass, most significant first) finds the K-th largest key T and how many
// keys equal to T are needed; an ordered compaction then emits every index whose key is > T and the
// lowest-index `need` entries whose key == T, in ascending index order. The result is therefore a
// deterministic function of the scores: ties on the K-th score go to the lowest indices.
#include <cooperative_groups.h>

#include "attn_state.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace djv {

constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / WARP;

// order-preserving map to unsigned; NaN (either sign) ranks above +inf, like torch.topk
__device__ __forceinline__ unsigned key_of(__half v) {
  unsigned short u = __half_as_ushort(v);
  if ((u & 0x7fffu) > 0x7c00u) return 0xffffu;
  if ((u & 0x7fffu) == 0) u = 0;  // -0.0 and +0.0 compare equal
  return (u & 0x8000u) ? (unsigned)(unsigned short)~u : (unsigned)(u | 0x8000u);
}
__device__ __forceinline__ unsigned key_of(float v) {
  unsigned u = __float_as_uint(v);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
  if ((u & 0x7fffffffu) == 0) u = 0;  // -0.0 and +0.0 compare equal
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
struct KeyTraits;
template <>
struct KeyTraits<__half> {
  using Key = unsigned short;
  static constexpr int BITS = 16;
};
template <>
struct KeyTraits<float> {
  using Key = unsigned;
  static constexpr int BITS = 32;
};

// exclusive block scan of one int per thread; returns the exclusive prefix, *total = block sum
__device__ __forceinline__ int block_exscan(int v, int *warp_sums, int *total) {
  const int lane = threadIdx.x % WARP, warp = threadIdx.x / WARP;
  int inc = v;
#pragma unroll
  for (int o = 1; o < WARP; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == WARP - 1) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < TK_WARPS) ? warp_sums[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < WARP; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < TK_WARPS) warp_sums[lane] = winc - w;  // exclusive warp offsets
    if (lane == WARP - 1) *total = winc;
  }
  __syncthreads();
  const int res = warp_sums[warp] + inc - v;
  __syncthreads();
  return res;
}

// Warp 0: given the histogram of the current 8 key bits over the candidates (keys that match `prefix` on the bits
// already fixed), find the bin that holds the need-th largest candidate; fixes those bits in *s_prefix and leaves
// in *s_need how many keys of that bin are still wanted.
__device__ __forceinline__ void select_bin(const int *hist, unsigned prefix, int need, int shift, unsigned *s_prefix,
                                           int *s_need) {
  const int tid = threadIdx.x;
  // lane l owns bins [8l, 8l+8); suffix counts from the top
  int c[8], sum = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    c[e] = hist[tid * 8 + e];
    sum += c[e];
  }
  // above = number of keys in bins owned by higher lanes
  int inc = sum;
#pragma unroll
  for (int o = 1; o < WARP; o <<= 1) {
    int t = __shfl_down_sync(0xffffffffu, inc, o);
    if (tid + o < WARP) inc += t;
  }
  int above = inc - sum;
  if (above < need && need <= above + sum) {
#pragma unroll
    for (int e = 7; e >= 0; --e) {
      if (above < need && need <= above + c[e]) {
        *s_prefix = prefix | ((unsigned)(tid * 8 + e) << shift);
        *s_need = need - above;
        above = need;  // stop
      } else {
        above += c[e];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(TK_THREADS)
topk_kernel(int32_t *__restrict__ idx32, int64_t *__restrict__ idx64, const T *__restrict__ scores,
            int n, int K, int n_sub, int *attn_state, int attn_nheads, int attn_S) {
  pdl_prologue();
  using Key = typename KeyTraits<T>::Key;
  constexpr int BITS = KeyTraits<T>::BITS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // [n_sub histograms of 256 counters][n keys]
  int *sub_hist = reinterpret_cast<int *>(smem_raw);
  Key *keys = reinterpret_cast<Key *>(smem_raw + (size_t)n_sub * 256 * sizeof(int));
  __shared__ int hist[256];
  __shared__ int warp_sums[TK_WARPS];
  __shared__ int s_total;
  __shared__ unsigned s_prefix;
  __shared__ int s_need;

  const int tid = threadIdx.x;
  for (int i = tid; i < n_sub * 256; i += TK_THREADS) sub_hist[i] = 0;
  for (int i = tid; i < n; i += TK_THREADS) keys[i] = (Key)key_of(scores[i]);
  if (tid == 0) {
    s_prefix = 0;
    s_need = K;
  }
  __syncthreads();

  unsigned mask = 0;
  for (int shift = BITS - 8; shift >= 0; shift -= 8) {
    const unsigned prefix = s_prefix;
    const int need = s_need;
    // Scores cluster in a few exponent bins, so all warps adding into one histogram would serialise on a
    // handful of shared-memory words: every group of warps counts into its own copy, added up afterwards.
    {
      int *my_hist = sub_hist + (tid / WARP % n_sub) * 256;
      for (int i = tid; i < n; i += TK_THREADS) {
        const unsigned k = keys[i];
        if ((k & mask) == prefix) atomicAdd(&my_hist[(k >> shift) & 0xffu], 1);
      }
    }
    __syncthreads();
    if (tid < 256) {
      int sum = 0;
      for (int c = 0; c < n_sub; ++c) {
        sum += sub_hist[c * 256 + tid];
        sub_hist[c * 256 + tid] = 0;
      }
      hist[tid] = sum;
    }
    __syncthreads();
    if (tid < WARP) select_bin(hist, prefix, need, shift, &s_prefix, &s_need);
    mask |= 0xffu << shift;
    __syncthreads();
  }

  const unsigned T_key = s_prefix;
  const int need = s_need;  // how many keys == T_key to take (lowest indices first)

  // ordered compaction: thread t owns the contiguous index range [t*per, (t+1)*per)
  const int per = (n + TK_THREADS - 1) / TK_THREADS;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  int gt = 0, eq = 0;
  for (int i = lo; i < hi; ++i) {
    const unsigned k = keys[i];
    gt += (k > T_key);
    eq += (k == T_key);
  }
  const int eq_before = block_exscan(eq, warp_sums, &s_total);
  int eq_take = need - eq_before;
  eq_take = eq_take < 0 ? 0 : (eq_take > eq ? eq : eq_take);
  int pos = block_exscan(gt + eq_take, warp_sums, &s_total);
  if (K > 0) {
    int taken_eq = 0;
    for (int i = lo; i < hi; ++i) {
      const unsigned k = keys[i];
      bool take = k > T_key;
      if (k == T_key && taken_eq < eq_take) {
        take = true;
        ++taken_eq;
      }
      if (take) {
        if (idx32) idx32[pos] = i;
        if (idx64) idx64[pos] = i;
        ++pos;
      }
    }
  }
  // the selection just made is the head list of an attention layer: open that layer's decode step here
  if (attn_state != nullptr) {
    __syncthreads();  // idx32 is complete and visible to the whole block
    attn_prep_block(attn_state, idx32, K, nullptr, nullptr, 0, attn_nheads, attn_S);
  }
}

// ---- long vectors: a cluster of 8 blocks -------------------------------------------------------------
// Block r holds the keys of the contiguous index range r * per_b .. in its shared memory. Every radix pass each
// block counts its own candidates, the 8 histograms are added through distributed shared memory by every block
// for itself (same numbers, same choice: no broadcast), and the compaction is ordered block by block, warp by warp,
// 32 indices at a time with ballots (the blocks exchange how many entries each emits): ascending index order, ties on the K-th score to the lowest indices, as in
// the one-block kernel.
constexpr int TC_THREADS = 512;
constexpr int TC_WARPS = TC_THREADS / WARP;
constexpr int TC_C = 8;    // blocks per cluster
constexpr int TC_SUB = 4;  // histogram copies per block

template <typename T>
__global__ void __cluster_dims__(TC_C, 1, 1) __launch_bounds__(TC_THREADS)
topk_cluster_kernel(int32_t *__restrict__ idx32, int64_t *__restrict__ idx64, const T *__restrict__ scores, int n,
                    int K, int per_b) {
  pdl_prologue();
  cg::cluster_group cluster = cg::this_cluster();
  using Key = typename KeyTraits<T>::Key;
  constexpr int BITS = KeyTraits<T>::BITS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Key *keys = reinterpret_cast<Key *>(smem_raw);
  __shared__ int sub_hist[TC_SUB][256];
  __shared__ int hist_pub[2][256];  // this block's histogram of a pass, read by the whole cluster
  __shared__ int hist[256];
  __shared__ int cnt_pub[2];        // this block's keys above / equal to the K-th key
  __shared__ int warp_gt[TC_WARPS], warp_eq[TC_WARPS];
  __shared__ unsigned s_prefix;
  __shared__ int s_need;

  const int tid = threadIdx.x, lane = tid % WARP, warp = tid / WARP;
  const int rank = (int)cluster.block_rank();
  const int b_lo = min(n, rank * per_b), b_hi = min(n, b_lo + per_b), nb = b_hi - b_lo;
  for (int i = tid; i < TC_SUB * 256; i += TC_THREADS) (&sub_hist[0][0])[i] = 0;
  for (int i = tid; i < nb; i += TC_THREADS) keys[i] = (Key)key_of(scores[b_lo + i]);
  if (tid == 0) {
    s_prefix = 0;
    s_need = K;
  }
  __syncthreads();

  unsigned mask = 0;
  int pass = 0;
  for (int shift = BITS - 8; shift >= 0; shift -= 8, ++pass) {
    const unsigned prefix = s_prefix;
    const int need = s_need;
    int *my_hist = sub_hist[warp % TC_SUB];
    for (int i = tid; i < nb; i += TC_THREADS) {
      const unsigned k = keys[i];
      if ((k & mask) == prefix) atomicAdd(&my_hist[(k >> shift) & 0xffu], 1);
    }
    __syncthreads();
    int *pub = hist_pub[pass & 1];  // (its readers of two passes ago are past the previous cluster barrier)
    if (tid < 256) {
      int sum = 0;
#pragma unroll
      for (int c = 0; c < TC_SUB; ++c) {
        sum += sub_hist[c][tid];
        sub_hist[c][tid] = 0;
      }
      pub[tid] = sum;
    }
    cluster.sync();
    if (tid < 256) {
      int sum = 0;
#pragma unroll
      for (int j = 0; j < TC_C; ++j) sum += cluster.map_shared_rank(pub, j)[tid];
      hist[tid] = sum;
    }
    __syncthreads();
    if (tid < WARP) select_bin(hist, prefix, need, shift, &s_prefix, &s_need);
    mask |= 0xffu << shift;
    __syncthreads();
  }
  const unsigned T_key = s_prefix;
  const int need = s_need;  // how many keys == T_key to take (lowest indices first)

  // warp w owns the chunks (32 consecutive indices) w * cpw .. of the block's range
  const int nchunks = (nb + WARP - 1) / WARP, cpw = (nchunks + TC_WARPS - 1) / TC_WARPS;
  const int c_lo = min(nchunks, warp * cpw), c_hi = min(nchunks, c_lo + cpw);
  int gt = 0, eq = 0;
  for (int c = c_lo; c < c_hi; ++c) {
    const int i = c * WARP + lane;
    const unsigned k = (i < nb) ? keys[i] : 0u;
    gt += __popc(__ballot_sync(0xffffffffu, i < nb && k > T_key));
    eq += __popc(__ballot_sync(0xffffffffu, i < nb && k == T_key));
  }
  if (lane == 0) {
    warp_gt[warp] = gt;
    warp_eq[warp] = eq;
  }
  __syncthreads();
  if (tid == 0) {
    int bgt = 0, beq = 0;
    for (int w = 0; w < TC_WARPS; ++w) {
      bgt += warp_gt[w];
      beq += warp_eq[w];
    }
    cnt_pub[0] = bgt;
    cnt_pub[1] = beq;
  }
  cluster.sync();
  // where this warp's first entry goes, and how many keys equal to the K-th key were taken before it
  int pos = 0, eq_seen = 0;
  auto skip = [&](int g, int e) {
    const int left = need - eq_seen;
    pos += g + (left < 0 ? 0 : (left > e ? e : left));
    eq_seen += e;
  };
  for (int j = 0; j < rank; ++j) {
    const int *c = cluster.map_shared_rank(cnt_pub, j);
    skip(c[0], c[1]);
  }
  cluster.barrier_arrive();  // this block has read its peers' shared memory for the last time
  for (int w = 0; w < warp; ++w) skip(warp_gt[w], warp_eq[w]);
  int eq_left = need - eq_seen;
  eq_left = eq_left < 0 ? 0 : eq_left;
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int c = c_lo; c < c_hi; ++c) {
    const int i = c * WARP + lane;
    const unsigned k = (i < nb) ? keys[i] : 0u;
    const bool g = i < nb && k > T_key, e = i < nb && k == T_key;
    const unsigned eb = __ballot_sync(0xffffffffu, e);
    const bool take = g || (e && __popc(eb & lt_mask) < eq_left);
    const unsigned tb = __ballot_sync(0xffffffffu, take);
    if (take) {
      const int p = pos + __popc(tb & lt_mask);
      if (idx32) idx32[p] = b_lo + i;
      if (idx64) idx64[p] = b_lo + i;
    }
    pos += __popc(tb);
    const int ne = __popc(eb);
    eq_left -= (ne < eq_left ? ne : eq_left);
  }
  cluster.barrier_wait();  // no block leaves while a peer may still read its counts
}

}  // namespace djv

using namespace djv;

static int launch_topk(int32_t *idx32, int64_t *idx64, const void *scores, int n, int K, int score_is_f32,
                       int *attn_state, int nheads, int S, cudaStream_t st) {
  // Long vectors that are not head lists: 8 blocks. (DJV_TK_CLUSTER_MIN: development knob, 0 = never.)
  static const int k_cluster_min = env_int("DJV_TK_CLUSTER_MIN", 4096);
  if (attn_state == nullptr && k_cluster_min > 0 && n >= k_cluster_min) {
    const int per_b = (n + TC_C - 1) / TC_C;
    const size_t smem = ((size_t)per_b * (score_is_f32 ? 4 : 2) + 15) & ~(size_t)15;
    if (smem <= 200 * 1024) {
      static const cudaError_t prep = [] {
        cudaError_t a = cudaFuncSetAttribute(topk_cluster_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             200 * 1024);
        cudaError_t b = cudaFuncSetAttribute(topk_cluster_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             200 * 1024);
        return a != cudaSuccess ? a : b;
      }();
      if (prep != cudaSuccess) {
        set_error("topk: cudaFuncSetAttribute: %s", cudaGetErrorString(prep));
        return DJV_ERR_CUDA;
      }
      if (score_is_f32)
        djv::launch_kernel(topk_cluster_kernel<float>, TC_C, TC_THREADS, smem, st, idx32, idx64,
                           static_cast<const float *>(scores), n, K, per_b);
      else
        djv::launch_kernel(topk_cluster_kernel<__half>, TC_C, TC_THREADS, smem, st, idx32, idx64,
                           static_cast<const __half *>(scores), n, K, per_b);
      count_launch();
      return check_launch("topk");
    }
  }
  const size_t bytes = (size_t)n * (score_is_f32 ? 4 : 2);
  if (bytes > 200 * 1024) {
    set_error("topk: n=%d scores (%zu bytes) exceed the 200 KiB shared-memory budget", n, bytes);
    return DJV_ERR_UNSUPPORTED;
  }
  // Four histogram copies (one per 8 warps). One per warp was measured slower inside a decode step: this
  // block shares its multiprocessor with blocks of the main chain, and the extra shared-memory traffic of
  // 32 copies slowed those down enough to stretch the kernels they belong to.
  static const int k_sub = env_int("DJV_TK_SUB", 4);  // development knob
  const int n_sub = (k_sub >= 1 && k_sub <= TK_WARPS) ? k_sub : 4;
  const size_t smem = ((bytes + 15) & ~(size_t)15) + (size_t)n_sub * 256 * sizeof(int);
  cudaError_t e;
  if (score_is_f32) {
    e = cudaFuncSetAttribute(topk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
    if (e == cudaSuccess)
      djv::launch_kernel(topk_kernel<float>, 1, TK_THREADS, smem, st, idx32, idx64,
                         static_cast<const float *>(scores), n, K, n_sub, attn_state, nheads, S);
  } else {
    e = cudaFuncSetAttribute(topk_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
    if (e == cudaSuccess)
      djv::launch_kernel(topk_kernel<__half>, 1, TK_THREADS, smem, st, idx32, idx64,
                         static_cast<const __half *>(scores), n, K, n_sub, attn_state, nheads, S);
  }
  if (e != cudaSuccess) {
    set_error("topk: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  count_launch();
  return check_launch("topk");
}

extern "C" int djv_topk(int32_t *idx32, int64_t *idx64, const void *scores, int n, int K,
                        int score_is_f32, void *stream) {
  DJV_REQUIRE(scores != nullptr, "topk: null scores");
  DJV_REQUIRE(n >= 1, "topk: n=%d", n);
  DJV_REQUIRE(K >= 0 && K <= n, "topk: K=%d outside [0,%d]", K, n);
  if (K == 0) return DJV_OK;
  DJV_REQUIRE(idx32 || idx64, "topk: no output pointer");
  return launch_topk(idx32, idx64, scores, n, K, score_is_f32, nullptr, 0, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int djv_topk_attn_prep(int32_t *idx32, const void *scores, int n, int K, int score_is_f32,
                                  int32_t *state, int S, void *stream) {
  DJV_REQUIRE(scores != nullptr && idx32 != nullptr && state != nullptr, "topk_attn_prep: null pointer");
  DJV_REQUIRE(n >= 1 && n <= 1024, "topk_attn_prep: %d heads outside [1,1024]", n);
  DJV_REQUIRE(K >= 1 && K <= n, "topk_attn_prep: K=%d outside [1,%d]", K, n);
  DJV_REQUIRE(S >= 1, "topk_attn_prep: cache capacity S=%d", S);
  return launch_topk(idx32, nullptr, scores, n, K, score_is_f32, state, n, S, static_cast<cudaStream_t>(stream));
}
