// Producer step in front of the decoder losses: per batch row, the K largest of F encoder
// activations, as int64 decoder-row indices plus values sorted in descending order -- exactly the
// (indices, vals) pair the loss kernels take.
//
// One CTA of 256 threads per row, several CTAs resident per SM, the row streamed from HBM ONCE:
//   1. every thread takes 16-byte vectors at a stride of the CTA and keeps running maxima of disjoint
//      element sets (packed NaN-propagating maxima, four instructions per vector): 1024 maxima per row
//      for fp32, 2048 for 16-bit types.  The K-th largest of them is a lower bound of the K-th largest
//      element, and for K << F a tight one (about 1.07 K elements reach it at K = 128, F = 65536);
//   2. that bound is found exactly on the top 16 bits of an order-preserving integer key (two 8-bit
//      histogram passes over the maxima, which never leave their registers);
//   3. the row is read again -- it is still in L2 -- and everything not below the bound is appended
//      to a candidate list in shared memory (any order);
//   4. the candidates are sorted by (key descending, index ascending) with a bitonic network and
//      the first K are the answer.
// The result is exact and independent of scheduling: the candidate SET is determined by the bound,
// and the sort is a total order.  Rows whose candidates overflow the list (masses of equal values,
// e.g. fewer than K positive entries after a ReLU) take an exact radix select over the whole row (8
// bits per pass on the full key, ties by ascending index) instead of step 3.
// NaN counts as larger than every number (as in torch.topk) and -0.0 equals +0.0.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

constexpr int kSelThreads = 256;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kSelMaxima = 4;                        // accumulators of running maxima per thread
constexpr int kSelMaxK = kSelThreads * kSelMaxima;   // the bound needs at least K maxima (16-bit types keep twice as many)
constexpr int kSelCandidates = 2048;                 // capacity of the candidate list (>= kSelMaxK)
constexpr int kSelInFlight = 8;                      // 16-byte loads in flight per thread
#ifndef FLEXSAE_SEL_MINB
#define FLEXSAE_SEL_MINB 4                           // resident CTAs per SM the kernel is compiled for
#endif

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

// bit pattern of element j of a 16-byte vector, as SelKey<T>::key takes it
template <typename T>
__device__ __forceinline__ uint32_t vector_bits(const uint4& v, int j) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if (SelKey<T>::BYTES == 4) return w[j];
  return (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
}

// Block-wide exclusive prefix sum (values stay below 2^31 in total); `total` receives the block
// total.  Ends with a barrier, so `scratch` (kSelWarps ints) may be reused at once.
__device__ __forceinline__ int sel_block_scan(int cnt, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  int before = incl - cnt, sum = 0;
#pragma unroll
  for (int w = 0; w < kSelWarps; w++) {
    const int t = scratch[w];
    if (w < warp) before += t;
    sum += t;
  }
  *total = sum;
  __syncthreads();
  return before;
}

// From a 256-bin histogram of the current digit (complete, a barrier behind it): the digit in which
// the `need`-th largest element lies and how many elements lie in higher digits.  Warp 0 works (8
// bins per lane, suffix sums by shuffles); everybody gets the answer.  Ends with a barrier.
__device__ __forceinline__ void sel_pick_digit(const int* hist, int* answer, int need, int* digit, int* above) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int h[8], mine = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      h[i] = hist[8 * lane + i];
      mine += h[i];
    }
    int incl = mine;  // inclusive suffix sum over lanes: bins of this lane and of all higher lanes
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int dn = __shfl_down_sync(0xffffffffu, incl, d);
      if (lane + d < 32) incl += dn;
    }
    int higher = incl - mine;  // elements in the bins of higher lanes
    if (incl >= need && higher < need) {  // exactly one lane: the suffix sums do not increase
#pragma unroll
      for (int i = 7; i >= 0; i--) {
        if (higher < need && higher + h[i] >= need) {
          answer[0] = 8 * lane + i;
          answer[1] = higher;
        }
        higher += h[i];
      }
    }
  }
  __syncthreads();
  *digit = answer[0];
  *above = answer[1];
  __syncthreads();
}

// one more element into a 256-bin histogram in shared memory; lanes of a warp that hit the same bin add
// once (the keys of a top-K problem crowd into very few bins).  bin < 0: nothing.  All 32 lanes call it.
__device__ __forceinline__ void sel_hist_add(int* hist, int bin) {
  const int lane = threadIdx.x & 31;
  const unsigned peers = __match_any_sync(0xffffffffu, bin < 0 ? -1 - lane : bin);
  if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(hist + bin, __popc(peers));
}

// ---- packed running maxima: the two passes over the row cost a handful of instructions per 16 bytes --
// A NaN must win (it ranks above every number), hence the NaN-propagating maxima.
template <typename T>
struct SelMax;
template <>
struct SelMax<float> {
  static constexpr int PER_ACC = 1;  // maxima held by one accumulator
  using acc_t = float;
  __device__ __forceinline__ static acc_t lowest() { return -INFINITY; }
  __device__ __forceinline__ static float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
  __device__ __forceinline__ static acc_t fold(acc_t a, const uint4& v) {
    return max_nan(max_nan(a, __uint_as_float(v.x)), max_nan(max_nan(__uint_as_float(v.y), __uint_as_float(v.z)), __uint_as_float(v.w)));
  }
  __device__ __forceinline__ static uint32_t bits(acc_t a, int) { return __float_as_uint(a); }
  // the largest element of one vector, as kept in shared memory between the two passes, and the
  // test "every element of that vector is below the bound" (false for a NaN on either side)
  using vmax_t = float;
  __device__ __forceinline__ static vmax_t vector_max(const uint4& v) { return fold(lowest(), v); }
  __device__ __forceinline__ static bool below(vmax_t m, float bound) { return m < bound; }
};
template <>
struct SelMax<__nv_bfloat16> {
  static constexpr int PER_ACC = 2;
  using acc_t = __nv_bfloat162;
  __device__ __forceinline__ static acc_t as2(uint32_t w) { return *reinterpret_cast<const __nv_bfloat162*>(&w); }
  __device__ __forceinline__ static acc_t lowest() { return as2(0xff80ff80u); }
  __device__ __forceinline__ static acc_t fold(acc_t a, const uint4& v) {
    return __hmax2_nan(__hmax2_nan(a, as2(v.x)), __hmax2_nan(__hmax2_nan(as2(v.y), as2(v.z)), as2(v.w)));
  }
  __device__ __forceinline__ static uint32_t bits(acc_t a, int i) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&a);
    return i ? (w >> 16) : (w & 0xffffu);
  }
  using vmax_t = __nv_bfloat16;
  __device__ __forceinline__ static vmax_t vector_max(const uint4& v) {
    const acc_t m = fold(lowest(), v);
    return __hmax_nan(__low2bfloat16(m), __high2bfloat16(m));
  }
  __device__ __forceinline__ static bool below(vmax_t m, float bound) { return __bfloat162float(m) < bound; }
};
template <>
struct SelMax<__half> {
  static constexpr int PER_ACC = 2;
  using acc_t = __half2;
  __device__ __forceinline__ static acc_t as2(uint32_t w) { return *reinterpret_cast<const __half2*>(&w); }
  __device__ __forceinline__ static acc_t lowest() { return as2(0xfc00fc00u); }
  __device__ __forceinline__ static acc_t fold(acc_t a, const uint4& v) {
    return __hmax2_nan(__hmax2_nan(a, as2(v.x)), __hmax2_nan(__hmax2_nan(as2(v.y), as2(v.z)), as2(v.w)));
  }
  __device__ __forceinline__ static uint32_t bits(acc_t a, int i) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&a);
    return i ? (w >> 16) : (w & 0xffffu);
  }
  using vmax_t = __half;
  __device__ __forceinline__ static vmax_t vector_max(const uint4& v) {
    const acc_t m = fold(lowest(), v);
    return __hmax_nan(__low2half(m), __high2half(m));
  }
  __device__ __forceinline__ static bool below(vmax_t m, float bound) { return __half2float(m) < bound; }
};

// KEEP_MAX: the maximum of every 16-byte vector is kept in (dynamic) shared memory during the first
// pass, so that the second pass touches only the few vectors that hold a candidate; without it (rows
// too long for that) the second pass reads the whole row again, from L2.
template <typename T, bool KEEP_MAX>
__global__ void __launch_bounds__(kSelThreads, FLEXSAE_SEL_MINB) topk_select_kernel(const SelectArgs a) {
  extern __shared__ __align__(16) unsigned char sel_dyn[];
  constexpr int VEC = Pack<T>::VEC;
  constexpr int NPASS = SelKey<T>::BYTES;
  constexpr int SHORT_SHIFT = 8 * NPASS - 16;  // the top 16 bits of a key are its "short key"
  constexpr int Q = kSelInFlight;
  __shared__ unsigned long long cand[kSelCandidates];  // (key << 32) | ~index; the whole-row select reuses it as histograms
  __shared__ int hist[256];
  __shared__ int misc[16];  // [0..1] digit / count above, [2] candidates so far, [8..15] scan scratch
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nvec = a.F / VEC;
  const uint4* row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.acts) + (size_t)blockIdx.x * a.F);

  // ---- 1. stream the row once: four accumulators of running maxima per thread (one per vector slot
  // modulo 4; a 16-bit accumulator holds two maxima, of the even and the odd elements)
  using Max = SelMax<T>;
  constexpr int NKEY = kSelMaxima * Max::PER_ACC;  // maxima per thread: disjoint element sets
  typename Max::vmax_t* vmax = reinterpret_cast<typename Max::vmax_t*>(sel_dyn);  // [nvec] when KEEP_MAX
  typename Max::acc_t top[kSelMaxima];
#pragma unroll
  for (int m = 0; m < kSelMaxima; m++) top[m] = Max::lowest();
  for (int base = 0; base < nvec; base += Q * kSelThreads) {
    uint4 x[Q];
#pragma unroll
    for (int q = 0; q < Q; q++) {
      const int v = base + q * kSelThreads + tid;
      if (v < nvec) x[q] = __ldg(row + v);
    }
#pragma unroll
    for (int q = 0; q < Q; q++) {
      const int v = base + q * kSelThreads + tid;
      if (v < nvec) {
        top[q % kSelMaxima] = Max::fold(top[q % kSelMaxima], x[q]);
        if (KEEP_MAX) vmax[v] = Max::vector_max(x[q]);  // read back by this same thread only
      }
    }
  }
  uint32_t skey[NKEY];  // short keys of the maxima (a set without elements ranks lowest: -inf)
#pragma unroll
  for (int m = 0; m < kSelMaxima; m++)
#pragma unroll
    for (int i = 0; i < Max::PER_ACC; i++) skey[m * Max::PER_ACC + i] = SelKey<T>::key(Max::bits(top[m], i)) >> SHORT_SHIFT;

  // ---- 2. K-th largest short key of the maxima (1024 or 2048 per row): two 8-bit histogram passes ----------------------
  int need = a.K, digit, above;
  hist[tid] = 0;
  if (tid == 0) misc[2] = 0;
  __syncthreads();
#pragma unroll
  for (int m = 0; m < NKEY; m++) sel_hist_add(hist, (int)(skey[m] >> 8));
  __syncthreads();
  sel_pick_digit(hist, misc, need, &digit, &above);
  need -= above;
  const uint32_t hi = (uint32_t)digit;
  hist[tid] = 0;
  __syncthreads();
#pragma unroll
  for (int m = 0; m < NKEY; m++) sel_hist_add(hist, (skey[m] >> 8) == hi ? (int)(skey[m] & 255u) : -1);
  __syncthreads();
  sel_pick_digit(hist, misc, need, &digit, &above);
  // lower edge of the short key's bin as a value: every element not below it is a candidate.  A bound
  // in the NaN range makes the comparison below true for everything: the row then overflows the list
  // and is selected exactly by the whole-row path.
  const uint32_t bound_key = ((hi << 8) | (uint32_t)digit) << SHORT_SHIFT;
  const float bound = SelKey<T>::value(bound_key);

  // ---- 3. candidates, appended in any order.  With the vector maxima at hand only the vectors that hold
  // a candidate are read again (a few hundred 16-byte loads per row, L2 hits); else the whole row is.
  auto take_from = [&](const uint4& x, int v) {
    float f[VEC];
    Pack<T>::unpack(x, f);
    unsigned hits = 0;
#pragma unroll
    for (int j = 0; j < VEC; j++) hits |= (unsigned)(!(f[j] < bound)) << j;  // a NaN is never below
    while (hits) {
      const int j = __ffs(hits) - 1;
      hits &= hits - 1;
      const int at = atomicAdd(&misc[2], 1);
      if (at < kSelCandidates)
        cand[at] = ((unsigned long long)SelKey<T>::key(vector_bits<T>(x, j)) << 32) | (uint32_t)~(uint32_t)(v * VEC + j);
    }
  };
  if (KEEP_MAX) {
    for (int v = tid; v < nvec; v += kSelThreads)
      if (!Max::below(vmax[v], bound)) take_from(__ldg(row + v), v);
  } else {
    for (int base = 0; base < nvec; base += Q * kSelThreads) {
      uint4 x[Q];
#pragma unroll
      for (int q = 0; q < Q; q++) {
        const int v = base + q * kSelThreads + tid;
        if (v < nvec) x[q] = __ldg(row + v);
      }
#pragma unroll
      for (int q = 0; q < Q; q++) {
        const int v = base + q * kSelThreads + tid;
        if (v < nvec && !Max::below(Max::vector_max(x[q]), bound)) take_from(x[q], v);
      }
    }
  }
  __syncthreads();
  int n_cand = misc[2];
  __syncthreads();

  if (n_cand > kSelCandidates) {
    // ---- 3b. too many candidates (masses of equal values): exact radix select over the whole row, 8
    // bits of the full key per pass, per-warp histograms; then the winners: everything above the K-th
    // key in any order, and of the elements equal to it the ones with the lowest indices
    int* warp_hist = reinterpret_cast<int*>(cand);  // [kSelWarps][256]
    uint32_t prefix = 0, hi_mask = 0;
    need = a.K;
    for (int pass = 0; pass < NPASS; pass++) {
      const int shift = 8 * (NPASS - 1 - pass);
      for (int i = tid; i < kSelWarps * 256; i += kSelThreads) warp_hist[i] = 0;
      __syncthreads();
      int* my_hist = warp_hist + warp * 256;
      for (int v0 = 0; v0 < nvec; v0 += kSelThreads) {  // uniform trip count: sel_hist_add needs whole warps
        const int v = v0 + tid;
        uint32_t k[VEC];
        if (v < nvec) vector_keys<T>(__ldg(row + v), k);
#pragma unroll
        for (int j = 0; j < VEC; j++)
          sel_hist_add(my_hist, (v < nvec && (k[j] & hi_mask) == prefix) ? (int)((k[j] >> shift) & 255u) : -1);
      }
      __syncthreads();
      int sum = 0;
      for (int w = 0; w < kSelWarps; w++) sum += warp_hist[w * 256 + tid];
      hist[tid] = sum;
      __syncthreads();
      sel_pick_digit(hist, misc, need, &digit, &above);
      prefix |= (uint32_t)digit << shift;
      need -= above;
      hi_mask |= 255u << shift;
    }
    const uint32_t kth = prefix;
    const int n_above = a.K - need;  // elements strictly above the K-th key: fewer than K
    if (tid == 0) misc[2] = 0;
    __syncthreads();  // the histograms are no longer read: the list may be written
    int tie_base = 0;
    for (int v0 = 0; v0 < nvec; v0 += kSelThreads) {
      const int v = v0 + tid;
      uint32_t k[VEC];
      int n_eq = 0;
      if (v < nvec) {
        vector_keys<T>(__ldg(row + v), k);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
          n_eq += k[j] == kth;
          if (k[j] > kth) cand[atomicAdd(&misc[2], 1)] = ((unsigned long long)k[j] << 32) | (uint32_t)~(uint32_t)(v * VEC + j);
        }
      }
      if (tie_base < need) {  // uniform: ties are taken in index order until `need` of them are in
        int total;
        int my_tie = tie_base + sel_block_scan(n_eq, misc + 8, &total);
        if (v < nvec) {
#pragma unroll
          for (int j = 0; j < VEC; j++)
            if (k[j] == kth) {
              if (my_tie < need) cand[n_above + my_tie] = ((unsigned long long)kth << 32) | (uint32_t)~(uint32_t)(v * VEC + j);
              my_tie++;
            }
        }
        tie_base += total;
      }
    }
    __syncthreads();
    n_cand = a.K;
  }

  // ---- 4. order: larger key first, equal keys by ascending index (entries are distinct: they carry
  // their index).  Short lists: every thread counts how many entries beat its own -- no barriers;
  // long lists: a bitonic network.
  const unsigned long long* sorted = cand;
  if (n_cand <= kSelThreads) {  // (longer lists: the network below does fewer comparisons)
    constexpr int kOut = kSelCandidates / 2;  // the ranked entries go to the upper half of the list
    const unsigned long long mine = tid < n_cand ? cand[tid] : 0ull;
    int rank = 0;
    for (int j = 0; j < n_cand; j++) rank += cand[j] > mine;
    if (tid < n_cand && rank < a.K) cand[kOut + rank] = mine;
    __syncthreads();
    sorted = cand + kOut;
  } else {
    int np = a.Kp;
    while (np < n_cand) np <<= 1;
    for (int i = n_cand + tid; i < np; i += kSelThreads) cand[i] = 0ull;  // padding sorts last
    __syncthreads();
    for (int k2 = 2; k2 <= np; k2 <<= 1) {
      for (int j = k2 >> 1; j > 0; j >>= 1) {
        for (int t = tid; t < (np >> 1); t += kSelThreads) {
          const int i = 2 * t - (t & (j - 1));  // the lower index of the t-th pair at distance j
          const int partner = i + j;
          const unsigned long long x = cand[i], y = cand[partner];
          const bool descending = (i & k2) == 0;
          if (descending ? x < y : x > y) {
            cand[i] = y;
            cand[partner] = x;
          }
        }
        __syncthreads();
      }
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
