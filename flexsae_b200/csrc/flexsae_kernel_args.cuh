// Compile-time constants, kernel argument blocks and staging helpers shared by the decoder-loss kernels.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

#ifndef FLEXSAE_CONVERT_BLOCKS
#define FLEXSAE_CONVERT_BLOCKS (148 * 3)
#endif
#ifndef FLEXSAE_CONVERT_IL
#define FLEXSAE_CONVERT_IL 4
#endif
#ifndef FLEXSAE_BWD_MINB
#define FLEXSAE_BWD_MINB 6  // resident CTAs per SM the backward is compiled for (register cap 80)
#endif
#ifndef FLEXSAE_FWD_MINB
#define FLEXSAE_FWD_MINB 6
#endif
constexpr int kThreads = 128;  // 4 warps per CTA: 16 / 8 / 4 lane groups for G = 8 / 16 / 32
constexpr int kUnroll = 8;     // decoder-row loads in flight per lane; segment lengths are multiples of it
constexpr int kRingSlots = 2 * kUnroll;  // backward: row pieces per lane in the shared-memory ring
__host__ __device__ constexpr int groups_per_cta(int G) { return kThreads / G; }

// Saved row state ("state" below), float32, written by the forward and read by the backward:
//   TopK          [B, D]            final residual (reconstruction - target)
//   Hierarchical  [2, NS, B, D]     part 0: residual after the last k of each K-segment,
//                                   part 1: running sum of the prefix residuals up to there.
// A K-segment is KS consecutive values of k (KS a multiple of kUnroll, NS = ceil(K / KS)).
// The backward of one batch row is independent per segment given these two vectors, which is
// what lets a small batch still fill the machine: suffix(k >= e) = total - running_sum(e - 1).
struct FwdArgs {
  const int64_t* indices;
  const void* weight;
  const void* vals;
  const void* bias;
  const void* target;
  float* loss_part;  // [pieces, B]
  float* state;
  int32_t* status;
  int B, K, F, D;
  int vals_dtype, bias_dtype, target_dtype;
  int KS, NS;
};

struct BwdArgs {
  const int64_t* indices;
  const void* weight;
  const void* vals;
  const float* state;
  const float* grad_out;  // device scalar
  float* slab;            // [F, PW] fp32 accumulation slab of this launch's column piece, zero on entry
  float* conv_slab;       // the other slab: finished piece `conv_piece`, converted by trailing CTAs
  void* dweight;          // [F, D] in the decoder's storage type
  float* dv_part;         // [pieces, B, K]
  float* s0;              // Hierarchical: [B, D] sum over k of the prefix residuals (dbias = coef * column sums)
  float* stage;           // deterministic mode: [B*K, PW] contribution rows in sorted-slot order
  const int* slot_of;     // deterministic mode: [B*K] sorted slot of each (b, k)
  int32_t* status;
  int B, K, F, D;
  int vals_dtype;
  int slab_stride; // floats between consecutive decoder rows of the accumulation target: PW (slab) or D (dweight itself)
  int piece;       // column piece accumulated by this launch (-1: none, conversion only)
  int conv_piece;  // column piece converted by this launch (-1: none)
  int unit_blocks; // CTAs that walk (row, segment) units
  int conv_blocks; // CTAs that convert; every conv_stride-th CTA of the grid until all are placed
  int conv_stride;
  float scale;     // 2 * inv_norm
  int KS, NS;
};

// One staged (index, value) pair: the index range-checked and narrowed, the value widened.
__device__ __forceinline__ int2 stage_pair(const int64_t* __restrict__ indices, const void* __restrict__ vals,
                                           int vals_dtype, size_t g, int F, int32_t* status) {
  int64_t x = indices[g];
  if ((uint64_t)x >= (uint64_t)F) {  // never dereference an index outside the table
    x = 0;
    if (status) atomicOr(status, FLEXSAE_STATUS_BAD_INDEX);
  }
  return make_int2((int)x, __float_as_int(load_scalar(vals, vals_dtype, g)));
}

template <int H>  // H float2 pairs = 2H floats, 16-byte aligned
__device__ __forceinline__ void load_pairs(const float* p, float2* out) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < H / 2; i++) {
    const float4 t = __ldg(q + i);
    out[2 * i] = make_float2(t.x, t.y);
    out[2 * i + 1] = make_float2(t.z, t.w);
  }
}

template <int H>
__device__ __forceinline__ void store_pairs(float* p, const float2* v) {
  float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
  for (int i = 0; i < H / 2; i++) q[i] = make_float4(v[2 * i].x, v[2 * i].y, v[2 * i + 1].x, v[2 * i + 1].y);
}

}  // namespace flexsae
