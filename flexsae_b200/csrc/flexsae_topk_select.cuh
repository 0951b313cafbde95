// Producer step in front of the decoder losses: per batch row, the K largest of F encoder
// activations, as int64 decoder-row indices plus values sorted in descending order -- exactly the
// (indices, vals) pair the loss kernels take.  One CTA per row.  The row is read from HBM once into
// shared memory when it fits (128 KB for F = 65536 in bf16) and every later pass runs out of shared
// memory; longer rows are re-read (they come back from L2).
//
// Selection is an exact radix select on an order-preserving integer key, 8 bits per pass from the
// top (2 passes for 16-bit activations, 4 for fp32): histogram of the current digit over the
// elements that still match the chosen prefix, suffix sums, pick the digit in which the K-th
// largest lies.  After the last pass the key of the K-th largest element is known exactly, and an
// index-ordered compaction takes everything above it plus the lowest-indexed ties, so the result
// does not depend on scheduling.  The K winners are then sorted (value descending, index ascending)
// with a bitonic network in shared memory.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

constexpr int kSelThreads = 1024;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kSelMaxK = 1024;
// shared memory besides the optional row cache: per-warp histograms (reused by the sort),
// the merged histogram and its suffix sums, scan scratch, a few scalars
constexpr size_t kSelFixedSmem = (size_t)kSelWarps * 256 * 4 + 256 * 4 * 2 + 64 * 4;

template <typename T>
struct SelKey;
template <>
struct SelKey<float> {
  static constexpr int BYTES = 4;
  __device__ __forceinline__ static uint32_t key(uint32_t u) { return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
  __device__ __forceinline__ static float value(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
  }
};
template <>
struct SelKey<__nv_bfloat16> {
  static constexpr int BYTES = 2;
  __device__ __forceinline__ static uint32_t key(uint32_t h) { return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u); }
  __device__ __forceinline__ static float value(uint32_t k) {
    const uint32_t h = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
    return __uint_as_float(h << 16);
  }
};
template <>
struct SelKey<__half> {
  static constexpr int BYTES = 2;
  __device__ __forceinline__ static uint32_t key(uint32_t h) { return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u); }
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

template <typename T, bool CACHED>
__global__ void __launch_bounds__(kSelThreads, 1) topk_select_kernel(const SelectArgs a) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int NPASS = SelKey<T>::BYTES;
  extern __shared__ uint4 sel_smem[];
  const int nvec = a.F / VEC;
  uint4* cache = sel_smem;
  int* warp_hist = reinterpret_cast<int*>(sel_smem + (CACHED ? nvec : 0));  // [warps][256]; later the sort buffer
  int* hist = warp_hist + kSelWarps * 256;                                  // [256]
  int* suffix = hist + 256;                                                 // [256]
  int* scratch = suffix + 256;                                              // [64]: warp totals, digit, count above
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint4* row = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.acts) + (size_t)blockIdx.x * a.F);

  if (CACHED) {
    for (int v = tid; v < nvec; v += kSelThreads) cache[v] = __ldcs(row + v);  // read once: streaming
    __syncthreads();
  }
  const uint4* src = CACHED ? cache : row;

  // ---- radix select: the key of the K-th largest element --------------------------------------
  uint32_t prefix = 0, hi_mask = 0;
  int need = a.K;  // how many of the elements matching `prefix` on the digits chosen so far are wanted
  for (int pass = 0; pass < NPASS; pass++) {
    const int shift = 8 * (NPASS - 1 - pass);
    for (int i = tid; i < kSelWarps * 256; i += kSelThreads) warp_hist[i] = 0;
    __syncthreads();
    int* mine = warp_hist + warp * 256;
    for (int v = tid; v < nvec; v += kSelThreads) {
      uint32_t k[VEC];
      vector_keys<T>(CACHED ? src[v] : __ldg(src + v), k);
#pragma unroll
      for (int j = 0; j < VEC; j++)
        if ((k[j] & hi_mask) == prefix) atomicAdd(mine + ((k[j] >> shift) & 255u), 1);
    }
    __syncthreads();
    if (tid < 256) {
      int s = 0;
      for (int w = 0; w < kSelWarps; w++) s += warp_hist[w * 256 + tid];
      hist[tid] = s;
      suffix[tid] = s;
    }
    __syncthreads();
    for (int d = 1; d < 256; d <<= 1) {  // suffix[i] = hist[i] + hist[i+1] + ... + hist[255]
      int add = 0;
      if (tid < 256 && tid + d < 256) add = suffix[tid + d];
      __syncthreads();
      if (tid < 256) suffix[tid] += add;
      __syncthreads();
    }
    if (tid < 256) {
      const int above = tid == 255 ? 0 : suffix[tid + 1];
      if (suffix[tid] >= need && above < need) {  // exactly one digit: the suffix sums do not increase
        scratch[32] = tid;
        scratch[33] = above;
      }
    }
    __syncthreads();
    prefix |= (uint32_t)scratch[32] << shift;
    need -= scratch[33];
    hi_mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t kth = prefix;       // key of the K-th largest
  const int n_above = a.K - need;    // elements strictly above it; `need` (>= 1) ties complete the K

  // ---- index-ordered compaction of the winners into the sort buffer -------------------------------
  unsigned long long* sorted = reinterpret_cast<unsigned long long*>(warp_hist);  // [Kp] (key << 32) | ~index
  for (int i = tid; i < a.Kp; i += kSelThreads) sorted[i] = 0ull;                 // padding sorts last
  __syncthreads();
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
    // block-wide exclusive scan of both counts at once (each below 2^16 per chunk)
    const uint32_t cnt = (uint32_t)n_gt | ((uint32_t)n_eq << 16);
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
    const uint32_t chunk_total = (uint32_t)scratch[kSelWarps - 1];
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
    above_base += (int)(chunk_total & 0xffffu);
    tie_base += (int)(chunk_total >> 16);
    __syncthreads();  // scratch is reused by the next chunk
  }

  // ---- bitonic sort, descending: larger key first, equal keys by ascending index ------------------
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
    if (a.relu) val = fmaxf(val, 0.f);
    store_scalar(a.vals, a.vals_dtype, (size_t)blockIdx.x * a.K + i, val);
    a.indices[(size_t)blockIdx.x * a.K + i] = (int64_t)(uint32_t)~(uint32_t)e;
  }
}

}  // namespace flexsae
