// Top-K index selection over one score vector, one block, keys held in shared memory.
//
// Radix select (8 bits per pass, most significant first) finds the K-th largest key T and how many
// keys equal to T are needed; an ordered compaction then emits every index whose key is > T and the
// lowest-index `need` entries whose key == T, in ascending index order. The result is therefore a
// deterministic function of the scores: ties on the K-th score go to the lowest indices.
#include "attn_state.cuh"
#include "common.cuh"

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
    // warp 0: find the bin holding the need-th largest key among the candidates
    if (tid < WARP) {
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
            s_prefix = prefix | ((unsigned)(tid * 8 + e) << shift);
            s_need = need - above;
            above = need;  // stop
          } else {
            above += c[e];
          }
        }
      }
    }
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

}  // namespace djv

using namespace djv;

static int launch_topk(int32_t *idx32, int64_t *idx64, const void *scores, int n, int K, int score_is_f32,
                       int *attn_state, int nheads, int S, cudaStream_t st) {
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
