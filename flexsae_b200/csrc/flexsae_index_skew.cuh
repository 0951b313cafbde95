// How unevenly indices[B,K] use the decoder rows: the largest number of sampled positions that name
// one row.  With heavily skewed indices (a Zipf law: a few decoder rows are named by nearly every
// batch row) the atomic backward is bound by the reductions into those rows, which serialise per
// 32-byte sector, and wide column pieces (which spread a hot row over more sectors at a time) win by
// 20-50 %; with uniform indices the narrower pieces that keep the fp32 slabs inside the L2 win.  The
// statistic lets a caller pick, without reading the indices on the host.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

constexpr int kSkewSamples = 65536;
constexpr int kSkewThreads = 256;

// histogram[F] and result[2] are zero on entry.  One thread per sampled position (an odd stride, so
// that with K a power of two the samples cover all K columns); the value an atomic increment returns, plus one, is a count
// some row reached, so the maximum over all threads is the largest count.
__global__ void __launch_bounds__(kSkewThreads)
index_skew_kernel(const long long* __restrict__ indices, long long n, long long stride, int samples, int F,
                  int* __restrict__ histogram, int* __restrict__ result) {
  const int i = blockIdx.x * kSkewThreads + threadIdx.x;
  int reached = 0;
  if (i < samples) {
    const long long f = indices[(long long)i * stride];
    if (f >= 0 && f < F) reached = atomicAdd(histogram + f, 1) + 1;
  }
  reached = __reduce_max_sync(0xffffffffu, reached);
  if ((threadIdx.x & 31) == 0 && reached > 0) atomicMax(result, reached);
  if (i == 0) result[1] = samples;
}

}  // namespace flexsae
