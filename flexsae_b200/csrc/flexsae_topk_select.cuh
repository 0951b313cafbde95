// Producer step in front of the decoder losses: per batch row, the K largest of F encoder
// activations, as int64 decoder-row indices plus values sorted in descending order -- exactly the
// (indices, vals) pair the loss kernels take.  One CTA per row.  The row is read from HBM once into
// shared memory when it fits (128 KB for F = 65536 in bf16) and every later pass runs out of shared
// memory; longer rows are re-read (they come back from L2).
//
// Selection is exact.  A pre-filter first bounds the answer from below: the K-th largest of the 1024
// per-thread maxima cannot exceed the K-th largest element, and for K << F barely more than K
// elements reach it (about 1.07 K for K = 128, F = 65536).  Those candidates are collected in index
// order, and a radix select on an order-preserving integer key (8 bits per pass from the top: 2
// passes for 16-bit activations, 4 for fp32) finds the key of the K-th largest among them;
// everything above it plus the lowest-indexed ties are the winners, so the result does not depend on
// scheduling.  Rows with masses of equal values overflow the candidate list and take the same radix
// select over the whole row instead.  The K winners are then sorted (value descending, index
// ascending) with a bitonic network in shared memory.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

constexpr int kSelThreads = 1024;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kSelMaxK = 1024;        // <= kSelThreads: the pre-filter needs at least K per-thread maxima
constexpr int kSelCandidates = 4096;  // capacity of the candidate list
// shared memory besides the optional row cache: candidate list (doubles as the per-warp histograms of
// the fallback), sort buffer, per-thread maxima, merged histogram and its suffix sums, scan scratch
constexpr size_t kSelFixedSmem =
    (size_t)kSelCandidates * 8 + (size_t)kSelMaxK * 8 + (size_t)kSelThreads * 4 + 256 * 4 * 2 + 64 * 4;

template <typename T>
struct SelKey;
template <>
struct SelKey<float> {
  static constexpr int BYTES = 4;
  __device__ __forceinline__ static uint32_t key(uint32_t u) {
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;  // NaN of either sign: above everything, like torch.topk
    if (u == 0x80000000u) u = 0u;                             // -0.0 ranks with +0.0 (they compare equal)
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
  __device__ __forceinline__ static float value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
  }
};
template <>
struct SelKey<__nv_bfloat16> {
  static constexpr int BYTES = 2;
  __device__ __forceinline__ static uint32_t key(uint32_t h) {
    if ((h & 0x7fffu) > 0x7f80u) return 0xffffu;  // NaN of either sign: above everything, like torch.topk
    if (h == 0x8000u) h = 0u;                     // -0.0 ranks with +0.0
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
  }
  __device__ __forceinline__ static float value(uint32_t k) {
    const uint32_t h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
    return __uint_as_float(h << 16);
  }
};
template <>
struct SelKey<__half> {
  static constexpr int BYTES = 2;
  __device__ __forceinline__ static uint32_t key(uint32_t h) {
    if ((h & 0x7fffu) > 0x7c00u) return 0xffffu;  // NaN of either sign: above everything
    if (h == 0x8000u) h = 0u;                     // -0.0 ranks with +0.0
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
  }
  __device__ __forceinline__ static float value(uint32_t k) {
    const uint32_t h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
    return __half2float(__ushort_as_half((unsigned short)h));
  }
};

// the VEC keys of one 16-byte vector, in element order
template <typename T>
__device__ __forceinline__ void vector_keys(const uint4& v, uint32_t* k) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (SelKey<T>::BYTES == 4) {
#pragma unroll
    for (int j = 0; j < 4; j++) k[j] = SelKey<T>::key(w[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      k[2 * j] = SelKey<T>::key(w[j] & 0xffffu);
      k[2 * j + 1] = SelKey<T>::key(w[j] >> 16);
    }
  }
}

struct SelectArgs {
  const void* acts;  // [B, F] activations
  void* vals;        // [B, K] out, vals_dtype
  int64_t* indices;  // [B, K] out
  int F, K, Kp;      // Kp = K rounded up to a power of two
  int vals_dtype;
  int relu;          // clamp the reported values at zero
};

// Block-wide exclusive prefix sum of a packed pair of counters (each field stays below 2^16 per
// call); `total` receives the block total.  Ends with a barrier, so `scratch` may be reused at once.
__device__ __forceinline__ uint32_t sel_block_scan(uint32_t cnt, int* scratch, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) scratch[warp] = (int)incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t t = (uint32_t)scratch[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, t, d);
      if (lane >= d) t += up;
    }
    scratch[lane] = (int)t;  // inclusive totals of the warps
  }
  __syncthreads();
  const uint32_t before = (warp ? (uint32_t)scratch[warp - 1] : 0u) + incl - cnt;
  *total = (uint32_t)scratch[kSelWarps - 1];
  __syncthreads();
  return before;
}

// From a merged 256-bin histogram of the current digit: the digit in which the `need`-th largest
// matching element lies, and how many matching elements lie in higher digits.
__device__ __forceinline__ void sel_pick_digit(int* hist, int* suffix, int* scratch, int need, int* digit, int* above) {
  const int tid = threadIdx.x;
  if (tid < 256) suffix[tid] = hist[tid];
  __syncthreads();
  for (int d = 1; d < 256; d <<= 1) {  // suffix[i] = hist[i] + hist[i+1] + ... + hist[255]
    int add = 0;
    if (tid < 256 && tid + d < 256) add = suffix[tid + d];
    __syncthreads();
    if (tid < 256) suffix[tid] += add;
    __syncthreads();
  }
  if (tid < 256) {
    const int up = tid == 255 ? 0 : suffix[tid + 1];
    if (suffix[tid] >= need && up < need) {  // exactly one digit: the suffix sums do not increase
      scratch[32] = tid;
      scratch[33] = up;
    }
  }
  __syncthreads();
  *digit = scratch[32];
  *above = scratch[33];
  __syncthreads();
}

// Exact radix select in a short list held in shared memory (the per-thread maxima, the candidate
// list): key of the `need`-th largest of `m` keys; *ties_needed = how many elements equal to it
// complete the selection.  Lanes that hit the same bin add once (match_any), because the keys of a
// top-K problem crowd into very few bins.
template <int NPASS, typename KeyAt>
__device__ __forceinline__ uint32_t sel_list_kth(KeyAt key_at, int m, int need, int* hist, int* suffix, int* scratch,
                                                 int* ties_needed) {
  const int tid = threadIdx.x, lane = tid & 31;
  uint32_t prefix = 0, hi_mask = 0;
  for (int pass = 0; pass < NPASS; pass++) {
    const int shift = 8 * (NPASS - 1 - pass);
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i0 = 0; i0 < m; i0 += kSelThreads) {
      const int i = i0 + tid;
      int bin = -1 - lane;  // lanes without a matching element: a value no other lane has
      if (i < m) {
        const uint32_t k = key_at(i);
        if ((k & hi_mask) == prefix) bin = (int)((k >> shift) & 255u);
      }
      const unsigned peers = __match_any_sync(0xffffffffu, bin);
      if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(hist + bin, __popc(peers));
    }
    __syncthreads();
    int digit, above;
    sel_pick_digit(hist, suffix, scratch, need, &digit, &above);
    prefix |= (uint32_t)digit << shift;
    need -= above;
    hi_mask |= 255u << shift;
  }
  *ties_needed = need;
  return prefix;
}

template <typename T, bool CACHED>
__global__ void __launch_bounds__(kSelThreads, 1) topk_select_kernel(const SelectArgs a) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int NPASS = SelKey<T>::BYTES;
  extern __shared__ uint4 sel_smem[];
  const int nvec = a.F / VEC;
  uint4* cache = sel_smem;
  unsigned long long* cand = reinterpret_cast<unsigned long long*>(sel_smem + (CACHED ? nvec : 0));  // [kSelCandidates]
  int* warp_hist = reinterpret_cast<int*>(cand);                     // fallback only: [warps][256], same memory
  unsigned long long* sorted = cand + kSelCandidates;                // [Kp] (key << 32) | ~index
  uint32_t* tmax = reinterpret_cast<uint32_t*>(sorted + kSelMaxK);   // [threads]
  int* hist = reinterpret_cast<int*>(tmax + kSelThreads);            // [256]
  int* suffix = hist + 256;                                          // [256]
  int* scratch = suffix + 256;                                       // [64]: warp totals, digit, count above
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint4* row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.acts) + (size_t)blockIdx.x * a.F);

  if (CACHED) {
    for (int v = tid; v < nvec; v += kSelThreads) cache[v] = __ldcs(row + v);  // read once: streaming
    __syncthreads();
  }
  const uint4* src = CACHED ? cache : row;

  // ---- 1. pre-filter.  The K-th largest of the per-thread maxima is a lower bound of the K-th
  // largest element (the K largest maxima are K different elements), and for K << F it is so tight
  // that barely more than K elements reach it.
  uint32_t mine = 0;  // key 0 is below every real key: the lowest one, that of -inf, is still positive
  for (int v = tid; v < nvec; v += kSelThreads) {
    uint32_t k[VEC];
    vector_keys<T>(CACHED ? src[v] : __ldg(src + v), k);
#pragma unroll
    for (int j = 0; j < VEC; j++) mine = max(mine, k[j]);
  }
  tmax[tid] = mine;
  for (int i = tid; i < a.Kp; i += kSelThreads) sorted[i] = 0ull;  // padding sorts last
  __syncthreads();
  int unused;
  const uint32_t bound = sel_list_kth<NPASS>([&](int i) { return tmax[i]; }, kSelThreads, a.K, hist, suffix, scratch, &unused);

  // ---- 2. candidates (key >= bound), collected in index order -----------------------------------
  int n_cand = 0;
  for (int v0 = 0; v0 < nvec; v0 += kSelThreads) {
    const int v = v0 + tid;
    uint32_t k[VEC];
    int n = 0;
    if (v < nvec) {
      vector_keys<T>(CACHED ? src[v] : __ldg(src + v), k);
#pragma unroll
      for (int j = 0; j < VEC; j++) n += k[j] >= bound;
    }
    uint32_t total;
    int at = n_cand + (int)sel_block_scan((uint32_t)n, scratch, &total);
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < VEC; j++)
        if (k[j] >= bound) {
          if (at < kSelCandidates) cand[at] = ((unsigned long long)k[j] << 32) | (uint32_t)~(uint32_t)(v * VEC + j);
          at++;
        }
    }
    n_cand += (int)total;
  }
  __syncthreads();

  if (n_cand <= kSelCandidates) {
    // ---- 3a. exact selection inside the candidate list, then the winners in list (= index) order
    int need;
    const uint32_t kth = sel_list_kth<NPASS>([&](int i) { return (uint32_t)(cand[i] >> 32); }, n_cand, a.K, hist, suffix,
                                             scratch, &need);
    const int n_above = a.K - need;
    int above_base = 0, tie_base = 0;
    for (int i0 = 0; i0 < n_cand; i0 += kSelThreads) {
      const int i = i0 + tid;
      const unsigned long long e = i < n_cand ? cand[i] : 0ull;
      const uint32_t k = (uint32_t)(e >> 32);
      const bool gt = i < n_cand && k > kth, eq = i < n_cand && k == kth;
      uint32_t total;
      const uint32_t before = sel_block_scan((uint32_t)gt | ((uint32_t)eq << 16), scratch, &total);
      if (gt) sorted[above_base + (int)(before & 0xffffu)] = e;
      if (eq && tie_base + (int)(before >> 16) < need) sorted[n_above + tie_base + (int)(before >> 16)] = e;
      above_base += (int)(total & 0xffffu);
      tie_base += (int)(total >> 16);
    }
  } else {
    // ---- 3b. fallback for rows with masses of equal values: radix select over the whole row, 8 bits
    // per pass, per-warp histograms; then the winners in index order
    uint32_t prefix = 0, hi_mask = 0;
    int need = a.K;
    for (int pass = 0; pass < NPASS; pass++) {
      const int shift = 8 * (NPASS - 1 - pass);
      for (int i = tid; i < kSelWarps * 256; i += kSelThreads) warp_hist[i] = 0;
      __syncthreads();
      int* my_hist = warp_hist + warp * 256;
      for (int v = tid; v < nvec; v += kSelThreads) {
        uint32_t k[VEC];
        vector_keys<T>(CACHED ? src[v] : __ldg(src + v), k);
#pragma unroll
        for (int j = 0; j < VEC; j++)
          if ((k[j] & hi_mask) == prefix) atomicAdd(my_hist + ((k[j] >> shift) & 255u), 1);
      }
      __syncthreads();
      if (tid < 256) {
        int sum = 0;
        for (int w = 0; w < kSelWarps; w++) sum += warp_hist[w * 256 + tid];
        hist[tid] = sum;
      }
      __syncthreads();
      int digit, above;
      sel_pick_digit(hist, suffix, scratch, need, &digit, &above);
      prefix |= (uint32_t)digit << shift;
      need -= above;
      hi_mask |= 255u << shift;
    }
    const uint32_t kth = prefix;
    const int n_above = a.K - need;
    int above_base = 0, tie_base = 0;
    for (int v0 = 0; v0 < nvec; v0 += kSelThreads) {
      const int v = v0 + tid;
      uint32_t k[VEC];
      int n_gt = 0, n_eq = 0;
      if (v < nvec) {
        vector_keys<T>(CACHED ? src[v] : __ldg(src + v), k);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
          n_gt += k[j] > kth;
          n_eq += k[j] == kth;
        }
      }
      uint32_t total;
      const uint32_t before = sel_block_scan((uint32_t)n_gt | ((uint32_t)n_eq << 16), scratch, &total);
      int my_above = above_base + (int)(before & 0xffffu);
      int my_tie = tie_base + (int)(before >> 16);
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < VEC; j++) {
          const unsigned long long entry = ((unsigned long long)k[j] << 32) | (uint32_t)~(uint32_t)(v * VEC + j);
          if (k[j] > kth) {
            sorted[my_above++] = entry;
          } else if (k[j] == kth) {
            if (my_tie < need) sorted[n_above + my_tie] = entry;
            my_tie++;
          }
        }
      }
      above_base += (int)(total & 0xffffu);
      tie_base += (int)(total >> 16);
    }
  }
  __syncthreads();

  // ---- 4. bitonic sort, descending: larger key first, equal keys by ascending index ---------------
  for (int k2 = 2; k2 <= a.Kp; k2 <<= 1) {
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < a.Kp; i += kSelThreads) {
        const int partner = i ^ j;
        if (partner > i) {
          const unsigned long long x = sorted[i], y = sorted[partner];
          const bool descending = (i & k2) == 0;
          if (descending ? x < y : x > y) {
            sorted[i] = y;
            sorted[partner] = x;
          }
        }
      }
      __syncthreads();
    }
  }
  for (int i = tid; i < a.K; i += kSelThreads) {
    const unsigned long long e = sorted[i];
    float val = SelKey<T>::value((uint32_t)(e >> 32));
    if (a.relu) val = val < 0.f ? 0.f : val;  // a NaN stays a NaN (fmaxf would hide it)
    store_scalar(a.vals, a.vals_dtype, (size_t)blockIdx.x * a.K + i, val);
    a.indices[(size_t)blockIdx.x * a.K + i] = (int64_t)(uint32_t)~(uint32_t)e;
  }
}

}  // namespace flexsae
