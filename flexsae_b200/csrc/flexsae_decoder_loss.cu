// Fused TopK / Hierarchical-TopK decoder loss for B200 (sm_100a): forward, backward and the
// C ABI around them.
//
// Work decomposition.  Everything in both losses is independent along the model width D except
// two reductions (the loss sum and the dvals dot products), so D is cut into column PIECES of
// PW = G * VEC columns (VEC = elements per 16-byte load, G = 8/16/32 lanes that share one batch
// row) and the grid is ordered piece-major: all batch rows for piece 0, then piece 1, ...
// While one piece is being processed, the only decoder bytes touched are that piece's columns
// of all F rows (F*PW*sizeof(T)), and the only gradient bytes touched are an fp32 slab
// [F, PW].  G is chosen so that both stay resident in the 126 MB L2: the K gathers of a batch
// row then hit L2 (each decoder row is used by many batch rows), and the dweight scatter-add is
// resolved by the L2 atomic units without read-modify-write traffic to HBM.  After a piece is
// done the slab is converted to the decoder's storage type, written to dweight and cleared.
//
// One lane group walks the K active rows of its batch row in order (forward) or in reverse
// (backward) with the running reconstruction in registers, so the [B, K, D] tensor of prefix
// reconstructions never exists.  This mirrors what hierarchical_sae_forward_kernel /
// hierarchical_sae_backward_kernel compute (torch-ext/flex_sae/hierarchical_kernels.py:12-187)
// and, with the prefix removed, embedding_bag_forward_kernel and the TopK gradient
// (torch-ext/flex_sae/topk_kernels.py:15-41,97-137).
#include <stdarg.h>

#include <mutex>
#include <stdio.h>
#include <string.h>

#include "flexsae_common.cuh"
#include "flexsae_deterministic.cuh"

namespace flexsae {

// ---- tuning state ------------------------------------------------------------------------------
struct Options {
  int lanes_fwd = 0;      // 0 = auto
  int lanes_bwd = 0;      // 0 = auto
  int l2_budget_mb = 80;  // one piece of decoder columns (+ one fp32 slab) must fit in this many MiB
  int segments = 0;       // K-segments per batch row in the backward; 0 = auto
  int pipeline = 1;       // 1: all column pieces of the atomic backward in one launch; 0: one launch per piece
  int convert_offset_pct = 60;  // where, inside a piece's unit blocks, the previous piece's converters sit
  int exchange_blocks = 148;    // sharded backward: blocks per slot for the cross-GPU reduce / broadcast / copy
  int direct_f32 = 1;           // fp32 decoder: reduce straight into dweight instead of slab + copy
};
static Options g_opt;

static thread_local char t_err[512] = "";
static thread_local int t_launches = 0;

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}

static size_t dtype_size(int dt) { return dt == FLEXSAE_F32 ? 4 : 2; }
static bool dtype_ok(int dt) { return dt == FLEXSAE_F32 || dt == FLEXSAE_BF16 || dt == FLEXSAE_F16; }
static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

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

__device__ __forceinline__ void load_f32(const float* p, float* out, int n4) {
  const float4* q = reinterpret_cast<const float4*>(p);
  for (int i = 0; i < n4; i++) {
    float4 t = __ldg(q + i);
    out[4 * i] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w;
  }
}

__device__ __forceinline__ void store_f32(float* p, const float* v, int n4) {
  float4* q = reinterpret_cast<float4*>(p);
  for (int i = 0; i < n4; i++) q[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
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

// ---- forward -----------------------------------------------------------------------------------
// SEG: the row is cut into several K-segments, so the residual and the running residual sum are
// saved at every segment end (otherwise only the final residual is saved).
template <typename T, int G, bool HIER, bool SEG>
__global__ void __launch_bounds__(kThreads, FLEXSAE_FWD_MINB) decoder_loss_fwd_kernel(const FwdArgs a) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int RPC = groups_per_cta(G);
  constexpr int U = kUnroll;
  constexpr int H = VEC / 2;
  extern __shared__ int2 staged[];  // [RPC][Kp]: (decoder-row offset in 16-byte units, vals bits)
  const int K = a.K;
  const int Kp = (K + U - 1) / U * U;  // padded to whole batches: padding = row 0 with vals 0
  const int row0 = blockIdx.x * RPC;
  const int piece = blockIdx.y;
  const uint32_t row16 = (uint32_t)(((size_t)a.D * sizeof(T)) >> 4);
  for (int i = threadIdx.x; i < RPC * Kp; i += kThreads) {
    const int lr = i / Kp;
    const int k = i - lr * Kp;
    const int b = row0 + lr;
    int2 e = make_int2(0, 0);
    if (b < a.B && k < K) {
      e = stage_pair(a.indices, a.vals, a.vals_dtype, (size_t)b * K + k, a.F, a.status);
      e.x = (int)((uint32_t)e.x * row16);
    }
    staged[i] = e;
  }
  __syncthreads();

  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int b = row0 + gid;
  const int col = piece * PW + lig * VEC;
  const bool active = (b < a.B) && (col < a.D);

  float2 r[H], acc[H], csum[H];
#pragma unroll
  for (int h = 0; h < H; h++) r[h] = acc[h] = csum[h] = make_float2(0.f, 0.f);
  if (active) {
    float bv[VEC], tv[VEC];
    load_elems<VEC>(a.bias, a.bias_dtype, (size_t)col, bv);
    load_elems<VEC>(a.target, a.target_dtype, (size_t)b * a.D + col, tv);
#pragma unroll
    for (int h = 0; h < H; h++) r[h] = make_float2(bv[2 * h] - tv[2 * h], bv[2 * h + 1] - tv[2 * h + 1]);
  }

  // lanes past the last column / row read column 0 of row 0 (valid memory) and never store
  const uint4* wcol = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(a.weight) +
                                                     (size_t)(active ? col : 0) * sizeof(T));
  const int2* mine = staged + gid * Kp;
  float* st_r = a.state + (size_t)b * a.D + col;                          // + s * B * D per segment
  float* st_c = st_r + (size_t)a.NS * a.B * a.D;
  const size_t seg_stride = (size_t)a.B * a.D;
  int seg = 0, seg_end = a.KS;

  for (int k0 = 0; k0 < Kp; k0 += U) {
    uint4 w[U];
    float v[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int2 e = mine[k0 + u];
      v[u] = __int_as_float(e.y);
      w[u] = ld_row_piece(wcol + (uint32_t)e.x);
    }
    const bool full = k0 + U <= K;
#pragma unroll
    for (int u = 0; u < U; u++) {
      const float2 vv = make_float2(v[u], v[u]);
      float2 wf[H];
      Pack<T>::unpack_pairs(w[u], wf);
      const bool real = full || (k0 + u < K);  // padding steps leave r unchanged (vals 0) but must not be penalised
#pragma unroll
      for (int h = 0; h < H; h++) {
        r[h] = fma2(vv, wf[h], r[h]);  // residual of the k-th prefix
        if (HIER && real) acc[h] = fma2(r[h], r[h], acc[h]);  // every prefix is penalised
        if (HIER && SEG && real) csum[h] = add2(csum[h], r[h]);
      }
    }
    if (HIER && SEG && (k0 + U == seg_end) && (k0 + U < K)) {  // a segment ends inside the row
      if (active) {
        store_pairs<H>(st_r + seg * seg_stride, r);
        store_pairs<H>(st_c + seg * seg_stride, csum);
      }
      seg++;
      seg_end += a.KS;
    }
  }
  if (!HIER) {
#pragma unroll
    for (int h = 0; h < H; h++) acc[h] = mul2(r[h], r[h]);
  }
  float s = 0.f;
#pragma unroll
  for (int h = 0; h < H; h++) s += acc[h].x + acc[h].y;
  if (!active) s = 0.f;  // lanes past the last column worked on column 0's data: not part of the loss
  s = group_sum<G>(s);
  if (lig == 0 && b < a.B) a.loss_part[(size_t)piece * a.B + b] = s;
  if (active) {
    store_pairs<H>(st_r + seg * seg_stride, r);  // HIER: seg == NS - 1 here; TopK: seg == 0
    if (HIER && SEG) store_pairs<H>(st_c + seg * seg_stride, csum);
  }
}

// Sum of the per-(piece, row) partial losses in a fixed order, in double, times the normaliser.
__global__ void __launch_bounds__(1024) loss_finalize_kernel(const float* __restrict__ part, size_t n, double inv_norm,
                                                             float* __restrict__ loss_out) {
  __shared__ double sh[1024];
  double s = 0.0;
  for (size_t i = threadIdx.x; i < n; i += 1024) s += (double)part[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int m = 512; m > 0; m >>= 1) {
    if ((int)threadIdx.x < m) sh[threadIdx.x] += sh[threadIdx.x + m];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss_out = (float)(sh[0] * inv_norm);
}

// ---- backward (atomic slab) ----------------------------------------------------------------------
// Sums each of 8 per-lane values over the G lanes of a group with 8 (G=16) shuffles instead of
// 8*log2(G): every exchange step halves the number of values a lane is responsible for.
// Returns, on every lane, the group total of value number (lig & 7).
template <int G>
__device__ __forceinline__ float group_sum8(const float* d, int lig) {
  float e[4], f[2];
  const bool b2 = lig & 4, b1 = lig & 2, b0 = lig & 1;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float send = b2 ? d[i] : d[i + 4];
    const float keep = b2 ? d[i + 4] : d[i];
    e[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const float send = b1 ? e[i] : e[i + 2];
    const float keep = b1 ? e[i + 2] : e[i];
    f[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  float g = (b0 ? f[1] : f[0]) + __shfl_xor_sync(0xffffffffu, b0 ? f[0] : f[1], 1);
#pragma unroll
  for (int m = 8; m < G; m <<= 1) g += __shfl_xor_sync(0xffffffffu, g, m);
  return g;
}

// fp32 slab -> the dweight columns of one piece in the decoder's storage type; clears the slab.
// Run by the trailing CTAs of the launch that accumulates the NEXT piece into the other slab,
// so the conversion streams through L2 while the atomic units are busy with that piece.
template <typename T, int G, bool L2_ONLY>
__device__ __forceinline__ void convert_slab(float* slab, void* __restrict__ dweight, int F, int D, int piece,
                                             int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = FLEXSAE_CONVERT_IL;  // independent items in flight per thread
  const size_t total = (size_t)F * G;
  const size_t stride = (size_t)nctas * kThreads;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    float4 lo[IL], hi[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        float* s = slab + (i / G) * PW + (i % G) * 4;
        // inside the single-launch pipeline the slab was last written by L2 atomics of the same
        // launch: read it at L2 (ld.cg), never through a possibly stale L1 line
        lo[q] = L2_ONLY ? __ldcg(reinterpret_cast<const float4*>(s)) : *reinterpret_cast<const float4*>(s);
        if (VEC == 8)
          hi[q] = L2_ONLY ? __ldcg(reinterpret_cast<const float4*>(s + G * 4)) : *reinterpret_cast<const float4*>(s + G * 4);
      }
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        const size_t f = i / G;
        const int lig = (int)(i % G);
        float* s = slab + f * PW + lig * 4;
        *reinterpret_cast<float4*>(s) = zero;
        float v[8] = {lo[q].x, lo[q].y, lo[q].z, lo[q].w, 0.f, 0.f, 0.f, 0.f};
        if (VEC == 8) {
          *reinterpret_cast<float4*>(s + G * 4) = zero;
          v[4] = hi[q].x; v[5] = hi[q].y; v[6] = hi[q].z; v[7] = hi[q].w;
        }
        const int col = piece * PW + lig * VEC;
        if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(dweight) + f * D + col) = Pack<T>::pack(v);
      }
    }
  }
}

// One step of the reverse walk for one lane: suffix += residual (skipped on padding steps),
// dweight contribution, dvals dot, residual stepped back to the previous prefix.
template <typename T, int G, bool HIER, bool DET, bool FULL>
__device__ __forceinline__ float walk_step(const int2 e, int slot, const uint4 piece16, bool in_seg, bool active, float coef,
                                           float2* r, float2* suf, float* slab, uint32_t slab_stride, float* stage) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int H = VEC / 2;
  constexpr int PW = G * VEC;
  const float v = __int_as_float(e.y);
  const float c = v * coef;
  const float2 cc = make_float2(c, c), nv = make_float2(-v, -v);
  float2 wf[H];
  Pack<T>::unpack_pairs(piece16, wf);
  if (HIER && (FULL || in_seg)) {
#pragma unroll
    for (int h = 0; h < H; h++) suf[h] = add2(suf[h], r[h]);  // S_k = sum_{j>=k} residual_j
  }
  if (active && (FULL || in_seg)) {
    float2 g[H];
#pragma unroll
    for (int h = 0; h < H; h++) g[h] = mul2(suf[h], cc);
    if (DET) {  // the contribution row goes to its sorted slot; it is added later, in slot order
      float4* dst = reinterpret_cast<float4*>(stage + (size_t)(uint32_t)slot * PW);
      __stcs(dst, make_float4(g[0].x, g[0].y, g[1].x, g[1].y));
      if (VEC == 8) __stcs(dst + 1, make_float4(g[H - 2].x, g[H - 2].y, g[H - 1].x, g[H - 1].y));
    } else {
      float* dst = slab + (size_t)((uint32_t)e.x) * slab_stride;
      red_add_v4(dst, g[0].x, g[0].y, g[1].x, g[1].y);
      if (VEC == 8) red_add_v4(dst + G * 4, g[H - 2].x, g[H - 2].y, g[H - 1].x, g[H - 1].y);
    }
  }
  float2 dot = make_float2(0.f, 0.f);
#pragma unroll
  for (int h = 0; h < H; h++) dot = fma2(wf[h], suf[h], dot);
  if (HIER) {
#pragma unroll
    for (int h = 0; h < H; h++) r[h] = fma2(nv, wf[h], r[h]);  // step back to prefix k-1 (v = 0 on padding)
  }
  return dot.x + dot.y;
}

// Slab column order: a lane's elements 0..3 live at column lig*4 and, for 8-element packs,
// elements 4..7 at column G*4 + lig*4, so that each red.v4 instruction of a lane group covers
// whole contiguous 32-byte sectors (a lane-contiguous 32-byte layout would make every sector
// the target of two separate instructions and halve the L2 atomic throughput).
//
// One lane group owns one (batch row, K-segment) unit and walks the segment from its last k
// down to its first: suffix += residual; dweight[idx] += vals * suffix; dvals = <row, suffix>;
// residual -= vals * row  (the reverse walk of hierarchical_kernels.py:147-173).
//
// The (decoder row, vals) pair of every (unit, step) is staged once per CTA (8 bytes; the sorted
// slot too in deterministic mode).  Padding steps (beyond K, or of a unit past the end) are staged
// as row 0 with vals = 0 and fetch zeros: they contribute exact zeros, and only the suffix update
// and the dvals store look at whether a step is real -- a whole batch of 8 real steps takes a path
// without those tests.
template <typename T, int G, bool HIER, bool DET>
__device__ __forceinline__ void walk_units(const BwdArgs& a, int unit_block, int piece, float* slab_base, uint4* smem) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int UPC = groups_per_cta(G);
  constexpr int U = kUnroll;
  constexpr int H = VEC / 2;
  static_assert(kRingSlots == 2 * kUnroll, "the ring holds the batch in use and the batch in flight");
  // Shared memory: a per-lane ring of 2*U row pieces (each lane only ever reads back the 16 bytes
  // it copied itself, so no warp synchronisation is involved), then the staged step records.
  uint4* ring = smem + threadIdx.x;  // slot s of this lane: ring[s * kThreads]
  int2* staged = reinterpret_cast<int2*>(smem + kRingSlots * kThreads);
  int* staged_slot = reinterpret_cast<int*>(staged + UPC * a.KS);  // deterministic mode only
  const int K = a.K, KS = a.KS, NS = a.NS;
  const int unit0 = unit_block * UPC;
  const int nunits = a.B * NS;
  const uint32_t row16 = (uint32_t)(((size_t)a.D * sizeof(T)) >> 4);  // decoder row length in 16-byte units
  for (int i = threadIdx.x; i < UPC * KS; i += kThreads) {
    const int lu = i / KS;
    const int j = i - lu * KS;
    const int u = unit0 + lu;
    int2 e = make_int2(0, 0);
    int slot = 0;
    if (u < nunits) {
      const int row = u / NS;
      const int k = (u - row * NS) * KS + j;
      if (k < K) {
        const size_t g = (size_t)row * K + k;
        e = stage_pair(a.indices, a.vals, a.vals_dtype, g, a.F, a.status);
        if (DET) slot = a.slot_of[g];
      }
    }
    staged[i] = e;
    if (DET) staged_slot[i] = slot;
  }
  __syncthreads();

  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int unit = unit0 + gid;
  const bool live = unit < nunits;
  const int row = live ? unit / NS : 0;
  const int seg = live ? unit - row * NS : 0;
  const int k_first = seg * KS;
  const int n = live ? min(KS, K - k_first) : 0;  // real steps of this segment
  const int col = piece * PW + lig * VEC;
  const bool active = live && (col < a.D);
  const float coef = __ldg(a.grad_out) * a.scale;

  float2 r[H], suf[H];
#pragma unroll
  for (int h = 0; h < H; h++) r[h] = suf[h] = make_float2(0.f, 0.f);
  if (active) {
    const size_t seg_stride = (size_t)a.B * a.D;
    const float* st = a.state + (size_t)row * a.D + col;
    load_pairs<H>(st + (HIER ? seg : 0) * seg_stride, r);
    if (!HIER) {
#pragma unroll
      for (int h = 0; h < H; h++) suf[h] = r[h];  // TopK: every k sees the same residual
    } else if (seg != NS - 1) {
      float2 c_here[H], c_all[H];
      load_pairs<H>(st + (size_t)(NS + seg) * seg_stride, c_here);
      load_pairs<H>(st + (size_t)(2 * NS - 1) * seg_stride, c_all);
#pragma unroll
      for (int h = 0; h < H; h++) suf[h] = make_float2(c_all[h].x - c_here[h].x, c_all[h].y - c_here[h].y);  // all later k
    }
  }

  // lanes past the last column read column 0 instead (valid memory); they never store or reduce
  const uint4* wcol = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(a.weight) +
                                                     (size_t)(active ? col : 0) * sizeof(T));
  const int2* mine = staged + gid * KS;
  const int* myslot = staged_slot + gid * KS;
  float* slab = slab_base + lig * 4;
  const uint32_t slab_stride = (uint32_t)a.slab_stride;
  float* stage = DET ? a.stage + lig * VEC : nullptr;
  float* dv = a.dv_part + ((size_t)piece * a.B + row) * K + k_first;

  // Row pieces travel global -> shared asynchronously through the ring: the piece for step
  // j - 16 is requested as soon as step j has been consumed, so a load is queued long BEFORE the
  // reductions of the steps in between (it does not sit behind them in the SM's memory pipeline)
  // and requests and reductions alternate instead of arriving in bursts.
  constexpr int R = kRingSlots;
  auto request = [&](int j, uint4* slot) {
    if (j >= 0) {  // padding steps and lanes past the last column get zeros without touching memory
      cp_async16(slot, wcol + (uint32_t)mine[j].x * row16, (active && j < n) ? 16 : 0);
    }
    cp_async_commit();  // one group per step (possibly empty) keeps the wait arithmetic uniform
  };
#pragma unroll
  for (int q = 0; q < R; q++) request(KS - 1 - q, ring + q * kThreads);
  int half = 0;
  for (int jb = KS - 1; jb >= 0; jb -= U, half ^= 1) {  // KS is a multiple of U
    uint4* slots = ring + half * U * kThreads;
    float d[U];
    if (jb < n) {  // all U steps are real
#pragma unroll
      for (int u = 0; u < U; u++) {
        cp_async_wait<R - 1>();  // at most R-1 newer requests pending: this step's piece has landed
        const uint4 w = slots[u * kThreads];
        request(jb - u - R, slots + u * kThreads);
        d[u] = walk_step<T, G, HIER, DET, true>(mine[jb - u], DET ? myslot[jb - u] : 0, w, true, active, coef, r, suf, slab,
                                                slab_stride, stage);
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; u++) {
        cp_async_wait<R - 1>();
        const uint4 w = slots[u * kThreads];
        request(jb - u - R, slots + u * kThreads);
        d[u] = walk_step<T, G, HIER, DET, false>(mine[jb - u], DET ? myslot[jb - u] : 0, w, jb - u < n, active, coef, r, suf,
                                                 slab, slab_stride, stage);
      }
    }
    const float tot = group_sum8<G>(d, lig);
    const int j = jb - (lig & 7);
    if (live && lig < 8 && j < n) dv[j] = tot * coef;
  }
  // The first segment ends with S_0, the sum of all prefix residuals of the row: dbias is the
  // column sum of these (TopK takes the column sums of the saved residual directly).
  if (HIER && active && seg == 0) store_pairs<H>(a.s0 + (size_t)row * a.D + col, suf);
}

// Multi-launch form: one launch per column piece; converting CTAs for the previous piece are
// spread evenly through the grid.
template <typename T, int G, bool HIER, bool DET>
__global__ void __launch_bounds__(kThreads, FLEXSAE_BWD_MINB) decoder_loss_bwd_kernel(const BwdArgs a) {
  extern __shared__ uint4 smem[];  // ring, staged pairs [UPC][KS], then (deterministic mode) int slots[UPC][KS]
  int unit_block = blockIdx.x;
  if (!DET && a.conv_blocks > 0) {
    const int q = blockIdx.x / a.conv_stride;
    if (q < a.conv_blocks && (int)blockIdx.x - q * a.conv_stride == a.conv_stride - 1) {
      convert_slab<T, G, false>(a.conv_slab, a.dweight, a.F, a.D, a.conv_piece, q, a.conv_blocks);
      return;
    }
    unit_block = blockIdx.x - min(q, a.conv_blocks);
  }
  walk_units<T, G, HIER, DET>(a, unit_block, a.piece, a.slab, smem);
}

// ---- single-launch pipelined backward ------------------------------------------------------------
// All column pieces in ONE grid, ordered piece by piece.  Piece p's blocks are its unit blocks
// with the blocks that convert piece p-1 inserted after the first quarter.  Two counters per
// piece carry the only dependencies:
//   converting blocks of piece q wait until all unit blocks of piece q have finished;
//   unit blocks of piece p wait until piece p-2 (same slab) has been converted and cleared.
// Every wait is on blocks with LOWER block indices, which the hardware dispatches first, so the
// lowest unfinished block never waits on anything unfinished.  Waits are bounded: after
// kSpinLimit polls a block gives up, sets FLEXSAE_STATUS_PIPELINE_TIMEOUT and carries on (the
// result is then invalid but the GPU is not held).
struct PipeArgs {
  BwdArgs b;
  float* slabs[2];
  int* walk_done;  // [pieces]
  int* conv_done;  // [pieces]
  int pieces, unit_blocks, conv_blocks, conv_offset;
};

constexpr int kSpinLimit = 1000000;  // polls of >= 0.2 us each: a fraction of a second

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void wait_count(const int* ctr, int target, int32_t* status) {
  if (threadIdx.x == 0) {
    int spins = 0;
    while (ld_acquire(ctr) < target) {
      __nanosleep(200);
      ++spins;
      // once any block has given up, nobody waits any more: the launch drains quickly
      const bool abandoned = status && (spins & 1023) == 0 &&
                             (*reinterpret_cast<volatile int32_t*>(status) & FLEXSAE_STATUS_PIPELINE_TIMEOUT);
      if (spins > kSpinLimit || abandoned) {
        if (status) atomicOr(status, FLEXSAE_STATUS_PIPELINE_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void signal_done(int* ctr) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();  // this block's reductions / stores are visible before the count moves
    atomicAdd(ctr, 1);
  }
}

template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(kThreads, FLEXSAE_BWD_MINB) decoder_loss_bwd_pipelined_kernel(const PipeArgs pa) {
  extern __shared__ uint4 smem[];
  const int per = pa.unit_blocks + pa.conv_blocks;
  const int p = blockIdx.x / per;
  const int r = blockIdx.x - p * per;
  int conv_idx = -1, unit_block = -1;
  if (p == pa.pieces) {
    conv_idx = r;  // the trailing blocks convert the last piece
  } else if (r >= pa.conv_offset && r < pa.conv_offset + pa.conv_blocks) {
    conv_idx = r - pa.conv_offset;
  } else {
    unit_block = r < pa.conv_offset ? r : r - pa.conv_blocks;
  }
  if (conv_idx >= 0) {
    const int q = p - 1;
    if (q < 0) return;
    wait_count(pa.walk_done + q, pa.unit_blocks, pa.b.status);
    convert_slab<T, G, true>(pa.slabs[q & 1], pa.b.dweight, pa.b.F, pa.b.D, q, conv_idx, pa.conv_blocks);
    signal_done(pa.conv_done + q);
    return;
  }
  if (pa.conv_blocks == 0) {
    // fp32 decoder: the reductions go straight into dweight's columns of this piece (cleared by
    // the caller); there is no slab, no conversion and nothing to wait for
    walk_units<T, G, HIER, false>(pa.b, unit_block, p, reinterpret_cast<float*>(pa.b.dweight) + (size_t)p * (G * Pack<T>::VEC),
                                  smem);
    return;
  }
  if (p >= 2) wait_count(pa.conv_done + (p - 2), pa.conv_blocks, pa.b.status);
  walk_units<T, G, HIER, false>(pa.b, unit_block, p, pa.slabs[p & 1], smem);
  signal_done(pa.walk_done + p);
}

// ---- batch-sharded backward: pipelined kernel + dweight reduction over peer memory ----------------
// Every rank (one GPU each, same node) runs this kernel on its own batch shard.  The converting
// blocks of the single-launch pipeline do the cross-GPU sum of dweight themselves, piece by piece,
// overlapped with the accumulation of the following pieces.  All traffic between GPUs is posted
// STORES into the peers' buffers (a remote load would stall its thread for microseconds; a store
// does not), all loads are local:
//   slot p converts the local slab of piece p-1 (decoder dtype) and SCATTERS it: every decoder row
//     goes to the inbox of the rank that owns that row block (reduce-scatter by push),
//   reduces piece p-2: this rank sums the N inbox copies of ITS row block (fixed rank order, fp32),
//     writes its own dweight rows and BROADCASTS the reduced rows into every peer's gather buffer,
//   copies piece p-3: the other ranks' reduced row blocks from the local gather buffer to dweight.
// One flag per (rank, peer) carries all cross-GPU ordering: when the last converting block of
// slot p finishes, the rank publishes seq_base + p to every rank; the converting blocks of slot p
// first wait until every rank (itself included) has published slot p-1.  Inbox and gather buffer
// are double-buffered by piece parity, and "every rank finished slot p-1" is exactly what makes a
// buffer complete to read and free to overwrite.  Waits are bounded like the local ones.  Plain
// peer stores only: no multicast of any kind.
constexpr int kMaxRanks = 8;
struct ShardArgs {
  PipeArgs p;
  int* slot_done;  // [pieces + 3] converting blocks that finished ALL stages of a slot
  int world, rank, rows_per_rank, seq_base;
  int exch_blocks;  // blocks per slot that reduce / broadcast / copy older pieces
  void* mc_inbox;     // multicast address of the inbox region of ALL ranks (NULL: plain peer stores)
  void* mc_gathered;  // multicast address of the gather buffers of all ranks
  void* inbox[kMaxRanks];    // rank o's inbox: [2][world][rows_per_rank][PW]
  void* gathered[kMaxRanks]; // rank o's gather buffer: [2][world * rows_per_rank][PW]
  int* flags_at[kMaxRanks];  // flag array living on rank s; entry [r] = last slot rank r finished
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void wait_peers(const ShardArgs& sa, int target) {
  if (threadIdx.x == 0) {
    int32_t* status = sa.p.b.status;
    const int* mine = sa.flags_at[sa.rank];
    for (int s = 0; s < sa.world; s++) {  // this rank too: its own earlier slot reads the buffers this slot rewrites
      int spins = 0;
      while (ld_acquire_sys(mine + s) - target < 0) {  // difference: robust to wrap-around
        __nanosleep(200);
        ++spins;
        const bool abandoned = status && (spins & 1023) == 0 &&
                               (*reinterpret_cast<volatile int32_t*>(status) & FLEXSAE_STATUS_PIPELINE_TIMEOUT);
        if (spins > kSpinLimit || abandoned) {
          if (status) atomicOr(status, FLEXSAE_STATUS_PIPELINE_TIMEOUT);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// local slab (fp32, permuted columns) -> decoder dtype, natural column order, each decoder row
// stored into the inbox of the rank owning its row block; clears the slab
template <typename T, int G>
__device__ __forceinline__ void slab_scatter(float* slab, const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = FLEXSAE_CONVERT_IL;
  const int F = sa.p.b.F;
  const int rpr = sa.rows_per_rank;
  const size_t total = (size_t)F * G;
  const size_t stride = (size_t)nctas * kThreads;
  const size_t slot_off = ((size_t)(piece & 1) * sa.world + sa.rank) * rpr * PW;  // [parity][sender = me]
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    float4 lo[IL], hi[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        float* sp = slab + (i / G) * PW + (i % G) * 4;
        lo[q] = __ldcg(reinterpret_cast<const float4*>(sp));
        if (VEC == 8) hi[q] = __ldcg(reinterpret_cast<const float4*>(sp + G * 4));
      }
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        const int f = (int)(i / G), lig = (int)(i % G);
        float* sp = slab + (size_t)f * PW + lig * 4;
        *reinterpret_cast<float4*>(sp) = zero;
        float v[8] = {lo[q].x, lo[q].y, lo[q].z, lo[q].w, 0.f, 0.f, 0.f, 0.f};
        if (VEC == 8) {
          *reinterpret_cast<float4*>(sp + G * 4) = zero;
          v[4] = hi[q].x; v[5] = hi[q].y; v[6] = hi[q].z; v[7] = hi[q].w;
        }
        const int owner = f / rpr;
        T* dst = reinterpret_cast<T*>(sa.inbox[owner]) + slot_off + (size_t)(f - owner * rpr) * PW + lig * VEC;
        *reinterpret_cast<uint4*>(dst) = Pack<T>::pack(v);  // a peer store unless this rank owns the row
      }
    }
  }
}

// this rank's row block of one piece: sum of the N inbox copies in rank order -> own dweight rows
// and every peer's gather buffer.  IL items per thread in flight (IL * world local 16-byte loads).
template <typename T, int G, int IL>
__device__ __forceinline__ void reduce_broadcast(const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int W = kMaxRanks / IL;  // largest world size this instantiation serves
  const int F = sa.p.b.F, D = sa.p.b.D;
  const int rpr = sa.rows_per_rank;
  const int row0 = sa.rank * rpr;
  const int rows = max(0, min(F, row0 + rpr) - row0);
  const size_t total = (size_t)rows * G;
  const size_t stride = (size_t)nctas * kThreads;
  const T* in = reinterpret_cast<const T*>(sa.inbox[sa.rank]) + (size_t)(piece & 1) * sa.world * rpr * PW;
  const size_t sender_stride = (size_t)rpr * PW;
  const size_t gat_off = ((size_t)(piece & 1) * sa.world * rpr + row0) * PW;
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    uint4 v[IL][W];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
#pragma unroll
      for (int s = 0; s < W; s++)
        if (i < total && s < sa.world) v[q][s] = __ldcg(reinterpret_cast<const uint4*>(in + s * sender_stride + i * VEC));
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[j] = 0.f;
#pragma unroll
        for (int s = 0; s < W; s++)
          if (s < sa.world) {
            float f[VEC];
            Pack<T>::unpack(v[q][s], f);
#pragma unroll
            for (int j = 0; j < VEC; j++) acc[j] += f[j];
          }
        const uint4 out = Pack<T>::pack(acc);
#pragma unroll
        for (int o = 0; o < kMaxRanks; o++)
          if (o < sa.world && o != sa.rank)
            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.gathered[o]) + gat_off + i * VEC) = out;  // peer store
        const int col = piece * PW + (int)(i % G) * VEC;
        if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.p.b.dweight) + (size_t)(row0 + i / G) * D + col) = out;
      }
    }
  }
}

// the other ranks' reduced row blocks of one piece: local gather buffer -> this rank's dweight
template <typename T, int G>
__device__ __forceinline__ void copy_gathered(const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = 8;
  const int F = sa.p.b.F, D = sa.p.b.D;
  const int rpr = sa.rows_per_rank;
  const size_t total = (size_t)F * G;  // items of the whole piece; this rank's own block is skipped
  const size_t stride = (size_t)nctas * kThreads;
  const T* src = reinterpret_cast<const T*>(sa.gathered[sa.rank]) + (size_t)(piece & 1) * sa.world * rpr * PW;
  const int own0 = sa.rank * rpr, own1 = own0 + rpr;
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    uint4 v[IL];
    bool take[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      const int f = (int)(i / G);
      take[q] = i < total && (f < own0 || f >= own1);
      if (take[q]) v[q] = __ldcg(reinterpret_cast<const uint4*>(src + i * VEC));
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      if (take[q]) {
        const size_t i = base + q * stride;
        const int col = piece * PW + (int)(i % G) * VEC;
        if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.p.b.dweight) + (i / G) * D + col) = v[q];
      }
    }
  }
}

// ---- the same three stages through the NVSwitch (multimem), when the buffers are bound to a
// multicast object: per GPU and step it moves F*D*sw bytes in each direction instead of
// 2*(N-1)/N times that, and a reduction is one load instead of N.
//   convert: slab -> this rank's OWN copy of the piece (region "inbox", used as [2][F][PW])
//   reduce:  multimem.ld_reduce of this rank's row block (the switch adds all ranks' copies in
//            fp32) -> own dweight rows + multimem.st into every rank's gather buffer
//   copy:    as before
template <typename T, int G>
__device__ __forceinline__ void slab_to_own_copy(float* slab, const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = FLEXSAE_CONVERT_IL;
  const int F = sa.p.b.F;
  const size_t total = (size_t)F * G;
  const size_t stride = (size_t)nctas * kThreads;
  T* x = reinterpret_cast<T*>(sa.inbox[sa.rank]) + (size_t)(piece & 1) * sa.world * sa.rows_per_rank * PW;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    float4 lo[IL], hi[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        float* sp = slab + (i / G) * PW + (i % G) * 4;
        lo[q] = __ldcg(reinterpret_cast<const float4*>(sp));
        if (VEC == 8) hi[q] = __ldcg(reinterpret_cast<const float4*>(sp + G * 4));
      }
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        float* sp = slab + (i / G) * PW + (i % G) * 4;
        *reinterpret_cast<float4*>(sp) = zero;
        float v[8] = {lo[q].x, lo[q].y, lo[q].z, lo[q].w, 0.f, 0.f, 0.f, 0.f};
        if (VEC == 8) {
          *reinterpret_cast<float4*>(sp + G * 4) = zero;
          v[4] = hi[q].x; v[5] = hi[q].y; v[6] = hi[q].z; v[7] = hi[q].w;
        }
        *reinterpret_cast<uint4*>(x + i * VEC) = Pack<T>::pack(v);
      }
    }
  }
}

template <typename T, int G>
__device__ __forceinline__ void switch_reduce_broadcast(const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = 8;  // switch reductions in flight per thread (each is a round trip through the NVSwitch)
  const int F = sa.p.b.F, D = sa.p.b.D;
  const int rpr = sa.rows_per_rank;
  const int row0 = sa.rank * rpr;
  const int rows = max(0, min(F, row0 + rpr) - row0);
  const size_t total = (size_t)rows * G;
  const size_t stride = (size_t)nctas * kThreads;
  const size_t par = (size_t)(piece & 1) * sa.world * rpr * PW;
  const T* mc_x = reinterpret_cast<const T*>(sa.mc_inbox) + par + (size_t)row0 * PW;
  T* mc_y = reinterpret_cast<T*>(sa.mc_gathered) + par + (size_t)row0 * PW;
  for (size_t base = (size_t)cta * kThreads + threadIdx.x; base < total; base += stride * IL) {
    uint4 v[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) v[q] = multimem_ld_reduce<T>(mc_x + i * VEC);
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = base + q * stride;
      if (i < total) {
        multimem_st(mc_y + i * VEC, v[q]);
        const int col = piece * PW + (int)(i % G) * VEC;
        if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.p.b.dweight) + (size_t)(row0 + i / G) * D + col) = v[q];
      }
    }
  }
}

// Block roles inside slot p of the sharded launch (slots 0..pieces+2):
//   exchange blocks (sa.exch_blocks, first in the slot): reduce + broadcast of piece p-2 and the
//     copy of piece p-3 -- local loads and posted stores only, so a few blocks keep up;
//   unit blocks: accumulate piece p;
//   converting blocks (inserted at conv_offset): slab of piece p-1 -> scattered to the owners, cleared.
// A slot is finished on a rank when all its exchange and converting blocks are.
template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(kThreads, FLEXSAE_BWD_MINB) decoder_loss_bwd_sharded_kernel(const ShardArgs sa) {
  extern __shared__ uint4 smem[];
  const PipeArgs& pa = sa.p;
  const int P = pa.pieces;
  const int E = sa.exch_blocks;
  const int per = E + pa.unit_blocks + pa.conv_blocks;
  const int body = P * per;
  int p, exch_idx = -1, conv_idx = -1, unit_block = -1;
  int exch_n = E;  // blocks that share the exchange work of this slot
  if ((int)blockIdx.x >= body) {  // three draining slots: no unit blocks, so every block helps with the exchange
    const int t = blockIdx.x - body;
    const int dper = E + pa.conv_blocks;
    p = P + t / dper;
    const int r = t - (p - P) * dper;
    if (p == P && r >= E) {
      conv_idx = r - E;  // slot P still has the last slab to convert
    } else {
      exch_idx = r;
      exch_n = (p == P) ? E : dper;
    }
  } else {
    p = blockIdx.x / per;
    int r = blockIdx.x - p * per;
    if (r < E) {
      exch_idx = r;
    } else {
      r -= E;
      if (r >= pa.conv_offset && r < pa.conv_offset + pa.conv_blocks) conv_idx = r - pa.conv_offset;
      else unit_block = r < pa.conv_offset ? r : r - pa.conv_blocks;
    }
  }
  if (unit_block >= 0) {
    if (p >= 2) wait_count(pa.conv_done + (p - 1), pa.conv_blocks, pa.b.status);  // slot p-1 cleared this slab
    walk_units<T, G, HIER, false>(pa.b, unit_block, p, pa.slabs[p & 1], smem);
    signal_done(pa.walk_done + p);
    return;
  }
  if (conv_idx >= 0) {
    if (p >= 1 && p - 1 < P) {
      wait_count(pa.walk_done + (p - 1), pa.unit_blocks, pa.b.status);  // the local slab is complete
      wait_peers(sa, sa.seq_base + p - 1);  // the owners have read what this parity of their inbox held
      if (sa.mc_inbox) slab_to_own_copy<T, G>(pa.slabs[(p - 1) & 1], sa, p - 1, conv_idx, pa.conv_blocks);
      else slab_scatter<T, G>(pa.slabs[(p - 1) & 1], sa, p - 1, conv_idx, pa.conv_blocks);
    }
    signal_done(pa.conv_done + p);
  } else {
    if (p >= 2) wait_peers(sa, sa.seq_base + p - 1);  // inbox of piece p-2 and gather buffer of piece p-3 are complete
    if (p >= 2 && p - 2 < P && sa.mc_inbox) {
      switch_reduce_broadcast<T, G>(sa, p - 2, exch_idx, exch_n);
    } else if (p >= 2 && p - 2 < P) {
      if (sa.world <= 2) reduce_broadcast<T, G, 4>(sa, p - 2, exch_idx, exch_n);
      else if (sa.world <= 4) reduce_broadcast<T, G, 2>(sa, p - 2, exch_idx, exch_n);
      else reduce_broadcast<T, G, 1>(sa, p - 2, exch_idx, exch_n);
    }
    if (p >= 3 && p - 3 < P) copy_gathered<T, G>(sa, p - 3, exch_idx, exch_n);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // this block's peer stores and dweight writes before the count moves
    const int old = atomicAdd(sa.slot_done + p, 1);
    if (old == E + pa.conv_blocks - 1) {  // the whole slot is done on this rank: tell every rank
      __threadfence_system();
      for (int s = 0; s < sa.world; s++) st_release_sys(sa.flags_at[s] + sa.rank, sa.seq_base + p);
    }
  }
}

// Column sums of a [B, D] fp32 matrix over row blocks: part[rb][d] = sum of rows of block rb.
// dbias is coef * (column sums of the final residual (TopK) / of the summed prefix residuals).
__global__ void __launch_bounds__(128) column_sums_kernel(const float* __restrict__ x, int B, int D, int rows_per_block,
                                                         float* __restrict__ part) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(B, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int q = 0; q < 8; q++) acc[q] = 0.f;
  for (int r = r0; r < r1; r += 8) {
#pragma unroll
    for (int q = 0; q < 8; q++)
      if (r + q < r1) acc[q] += x[(size_t)(r + q) * D + d];
  }
  part[(size_t)blockIdx.y * D + d] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

// dvals = sum over column pieces (fixed order), dbias = coef * sum over row blocks (fixed order).
__global__ void __launch_bounds__(256) grads_finalize_kernel(const float* __restrict__ dv_part, int pieces, size_t BK,
                                                            void* __restrict__ dvals, int vals_dtype,
                                                            const float* __restrict__ db_part, int row_blocks, int D,
                                                            void* __restrict__ dbias, int bias_dtype, int dv_blocks,
                                                            const float* __restrict__ grad_out, float scale) {
  if ((int)blockIdx.x < dv_blocks) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < BK) {
      float s = 0.f;
      for (int p = 0; p < pieces; p++) s += dv_part[(size_t)p * BK + i];
      store_scalar(dvals, vals_dtype, i, s);
    }
  } else {
    const int d = (blockIdx.x - dv_blocks) * blockDim.x + threadIdx.x;
    if (d < D) {
      float s = 0.f;
      for (int t = 0; t < row_blocks; t++) s += db_part[(size_t)t * D + d];
      store_scalar(dbias, bias_dtype, (size_t)d, s * (__ldg(grad_out) * scale));
    }
  }
}

// ---- host side -------------------------------------------------------------------------------------
struct Shape {
  int64_t B, K, F, D;
};

static int check_shape(int kind, const Shape& s, int wdt) {
  if (kind != FLEXSAE_TOPK && kind != FLEXSAE_HIER) return fail(FLEXSAE_EINVAL, "unknown loss kind %d", kind);
  if (!dtype_ok(wdt)) return fail(FLEXSAE_EINVAL, "unknown weight dtype code %d", wdt);
  if (s.B < 1 || s.K < 1 || s.F < 1 || s.D < 1)
    return fail(FLEXSAE_EINVAL, "B, K, F, D must be positive (got %lld %lld %lld %lld)", (long long)s.B, (long long)s.K,
                (long long)s.F, (long long)s.D);
  const int vec = 16 / (int)dtype_size(wdt);
  if (s.D % vec != 0)
    return fail(FLEXSAE_EUNSUPPORTED, "D=%lld must be a multiple of %d (16-byte row pieces)", (long long)s.D, vec);
  if (s.F > (1ll << 30) || s.D > (1ll << 20) || s.B > (1ll << 27) || s.B * s.K > (1ll << 31) - 1)
    return fail(FLEXSAE_EUNSUPPORTED, "shape too large for 32-bit row/position arithmetic");
  // 8 (+4 in deterministic mode) bytes per (unit, step) are staged in shared memory next to the
  // 32 KiB row-piece ring: 16 units * K * 12 bytes must fit
  if (s.K > 960) return fail(FLEXSAE_EUNSUPPORTED, "K=%lld above the supported maximum of 960", (long long)s.K);
  return 0;
}

// lanes per batch row: the widest group whose per-piece working set fits the L2 budget
static int choose_lanes(int64_t F, int wdt, bool with_slab, int forced) {
  if (forced == 8 || forced == 16 || forced == 32) return forced;
  const int vec = 16 / (int)dtype_size(wdt);
  const double budget = (double)g_opt.l2_budget_mb * 1048576.0;
  for (int G = 32; G >= 8; G >>= 1) {
    double bytes = (double)F * G * vec * (dtype_size(wdt) + (with_slab ? 4.0 : 0.0));
    if (bytes <= budget) return G;
  }
  return 32;  // nothing fits: stream from HBM with the widest (most coalesced) row pieces
}

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

// segment length for a requested number of K-segments, and the count that length gives
static void segment_layout(int K, int want, int* KS, int* NS) {
  if (want < 1) want = 1;
  int ks = round_up((K + want - 1) / want, kUnroll);
  *KS = ks;
  *NS = (K + ks - 1) / ks;
}

// K-segments so that one column piece of the backward offers about a full machine of warps
static int choose_segments(const Shape& s, int wdt) {
  int want = g_opt.segments;
  if (want <= 0) {
    const int G = choose_lanes(s.F, wdt, true, g_opt.lanes_bwd);
    const double warps = (double)s.B * G / 32.0;
    const double target = 148.0 * 32.0;
    want = (int)((target + warps - 1) / warps);
    if (want > 8) want = 8;
  }
  int KS, NS;
  segment_layout((int)s.K, want, &KS, &NS);
  if (g_opt.segments <= 0 && (long long)NS * KS != s.K) {
    // prefer the next larger count whose segments tile K exactly: padding steps are wasted work
    for (int w = want + 1; w <= 8; w++) {
      int ks, ns;
      segment_layout((int)s.K, w, &ks, &ns);
      if ((long long)ns * ks == s.K) return ns;
    }
  }
  return NS;
}

static size_t state_floats(int kind, const Shape& s, int NS) {
  return (size_t)s.B * s.D * ((kind == FLEXSAE_HIER && NS > 1) ? 2 * (size_t)NS : 1);
}

static int check_segments(int kind, const Shape& s, int segments, int* KS, int* NS) {
  if (segments < 1) return fail(FLEXSAE_EINVAL, "segments must be >= 1 (got %d)", segments);
  segment_layout((int)s.K, segments, KS, NS);
  if (*NS != segments)
    return fail(FLEXSAE_EINVAL, "segments=%d is not a layout of K=%lld (use flexsae_choose_segments; nearest is %d)",
                segments, (long long)s.K, *NS);
  return 0;
}

constexpr int kMaxRowBlocks = 128;  // partial rows of the dbias column sums
constexpr int kConvertBlocks = FLEXSAE_CONVERT_BLOCKS;  // CTAs per piece that convert the previous piece's slab

struct BwdPlan {
  int G, PW, pieces, row_blocks, rows_per_block;
  size_t slab_bytes, off_slab, off_dv, off_db, off_s0, off_ctr, off_index, off_stage, off_part, total;
};

static BwdPlan plan_bwd(const Shape& s, int wdt, int dw_mode) {
  BwdPlan p;
  const int vec = 16 / (int)dtype_size(wdt);
  p.G = choose_lanes(s.F, wdt, true, g_opt.lanes_bwd);
  p.PW = p.G * vec;
  p.pieces = (int)((s.D + p.PW - 1) / p.PW);
  p.rows_per_block = (int)((s.B + kMaxRowBlocks - 1) / kMaxRowBlocks);
  if (p.rows_per_block < 32) p.rows_per_block = 32;
  p.row_blocks = (int)((s.B + p.rows_per_block - 1) / p.rows_per_block);
  size_t off = 0;
  p.off_slab = off;  // two slabs: one accumulating, one being converted
  p.slab_bytes = dw_mode == FLEXSAE_DW_ATOMIC ? align_up((size_t)s.F * p.PW * 4, 256) : 0;
  off += 2 * p.slab_bytes;
  p.off_index = p.off_stage = p.off_part = off;
  if (dw_mode == FLEXSAE_DW_DETERMINISTIC) {
    const int64_t n = s.B * s.K;
    off += det_index_bytes(n, s.F);
    p.off_stage = off;
    off = align_up(off + (size_t)n * p.PW * 4, 256);
    p.off_part = off;
    off = align_up(off + det_part_rows(n, s.F) * p.PW * 4, 256);
  }
  p.off_dv = off;
  off = align_up(off + (size_t)p.pieces * s.B * s.K * 4, 256);
  p.off_db = off;
  off = align_up(off + (size_t)p.row_blocks * s.D * 4, 256);
  p.off_s0 = off;  // summed prefix residuals of every row (Hierarchical; TopK does not use it)
  off = align_up(off + (size_t)s.B * s.D * 4, 256);
  p.off_ctr = off;  // per-piece completion counters of the single-launch pipeline
  off = align_up(off + (size_t)(3 * p.pieces + 6) * 4, 256);
  p.total = off;
  return p;
}

struct FwdPlan {
  int G, PW, pieces;
  size_t total;
};

static FwdPlan plan_fwd(const Shape& s, int wdt) {
  FwdPlan p;
  const int vec = 16 / (int)dtype_size(wdt);
  p.G = choose_lanes(s.F, wdt, false, g_opt.lanes_fwd);
  p.PW = p.G * vec;
  p.pieces = (int)((s.D + p.PW - 1) / p.PW);
  p.total = align_up((size_t)p.pieces * s.B * 4, 256);
  return p;
}

constexpr size_t kRingBytes = (size_t)kRingSlots * kThreads * sizeof(uint4);  // 2 KiB per slot and CTA

template <typename K>
static cudaError_t allow_smem(K kern, size_t smem) {
  if (smem <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

template <typename T, int G, bool HIER, bool SEG>
static cudaError_t launch_fwd_seg(const FwdArgs& a, int pieces, cudaStream_t st) {
  constexpr int RPC = groups_per_cta(G);
  const size_t smem = (size_t)RPC * ((a.K + kUnroll - 1) / kUnroll * kUnroll) * sizeof(int2);
  auto kern = decoder_loss_fwd_kernel<T, G, HIER, SEG>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  dim3 grid((a.B + RPC - 1) / RPC, pieces);
  kern<<<grid, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_fwd(const FwdArgs& a, int pieces, cudaStream_t st) {
  if (HIER && a.NS > 1) return launch_fwd_seg<T, G, HIER, true>(a, pieces, st);
  return launch_fwd_seg<T, G, HIER, false>(a, pieces, st);
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_det(BwdArgs a, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * a.KS * (sizeof(int2) + sizeof(int));
  auto kern = decoder_loss_bwd_kernel<T, G, HIER, true>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  const long long units = (long long)a.B * a.NS;
  a.unit_blocks = (int)((units + UPC - 1) / UPC);
  a.conv_blocks = 0;
  a.conv_stride = 1;
  kern<<<a.unit_blocks, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd(BwdArgs a, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * a.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_kernel<T, G, HIER, false>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  const long long units = (long long)a.B * a.NS;
  a.unit_blocks = a.piece >= 0 ? (int)((units + UPC - 1) / UPC) : 0;
  int conv_blocks = 0;
  if (a.conv_piece >= 0) {
    const long long items = (long long)a.F * G;
    conv_blocks = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
    const int cap = a.piece >= 0 ? kConvertBlocks : kConvertBlocks * 4;
    if (conv_blocks > cap) conv_blocks = cap;
  }
  a.conv_blocks = conv_blocks;
  a.conv_stride = conv_blocks > 0 ? (a.unit_blocks + conv_blocks) / conv_blocks : 1;
  kern<<<a.unit_blocks + conv_blocks, kThreads, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_pipelined(const BwdArgs& b, float* slab0, float* slab1, int* counters, int pieces,
                                        bool direct, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * b.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_pipelined_kernel<T, G, HIER>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  PipeArgs pa;
  pa.b = b;
  pa.slabs[0] = slab0;
  pa.slabs[1] = slab1;
  pa.walk_done = counters;
  pa.conv_done = counters + pieces;
  pa.pieces = pieces;
  const long long units = (long long)b.B * b.NS;
  pa.unit_blocks = (int)((units + UPC - 1) / UPC);
  const long long items = (long long)b.F * G;
  int conv = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
  if (conv > kConvertBlocks) conv = kConvertBlocks;
  if (direct) conv = 0;
  pa.conv_blocks = conv;
  pa.conv_offset = (int)((long long)pa.unit_blocks * g_opt.convert_offset_pct / 100);
  const long long blocks = (long long)pieces * (pa.unit_blocks + conv) + conv;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kThreads, smem, st>>>(pa);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd_sharded(const BwdArgs& b, float* slab0, float* slab1, int* counters, int pieces,
                                      ShardArgs sa, cudaStream_t st) {
  constexpr int UPC = groups_per_cta(G);
  const size_t smem = kRingBytes + (size_t)UPC * b.KS * sizeof(int2);
  auto kern = decoder_loss_bwd_sharded_kernel<T, G, HIER>;
  if (cudaError_t e = allow_smem(kern, smem)) return e;
  PipeArgs& pa = sa.p;
  pa.b = b;
  pa.slabs[0] = slab0;
  pa.slabs[1] = slab1;
  pa.walk_done = counters;
  pa.conv_done = counters + pieces;       // one counter per slot: pieces + 3 of them
  sa.slot_done = counters + 2 * pieces + 3;  // and pieces + 3 more
  pa.pieces = pieces;
  const long long units = (long long)b.B * b.NS;
  pa.unit_blocks = (int)((units + UPC - 1) / UPC);
  const long long items = (long long)b.F * G;
  int conv = (int)((items + kThreads * 4 - 1) / (kThreads * 4));
  if (conv > kConvertBlocks) conv = kConvertBlocks;
  pa.conv_blocks = conv;
  pa.conv_offset = (int)((long long)pa.unit_blocks * g_opt.convert_offset_pct / 100);
  sa.exch_blocks = g_opt.exchange_blocks;
  const long long blocks = (long long)pieces * (sa.exch_blocks + pa.unit_blocks + conv) + 3ll * (sa.exch_blocks + conv);
  if (blocks > 0x7fffffffll) return cudaErrorInvalidConfiguration;
  kern<<<(unsigned)blocks, kThreads, smem, st>>>(sa);
  t_launches++;
  return cudaGetLastError();
}

// dispatch over (element type, lanes, loss kind)
#define FLEXSAE_DISPATCH_G(T, G, kind, CALL) ((kind) == FLEXSAE_HIER ? CALL(T, G, true) : CALL(T, G, false))
#define FLEXSAE_DISPATCH_T(T, G, kind, CALL)                                                       \
  ((G) == 32 ? FLEXSAE_DISPATCH_G(T, 32, kind, CALL)                                               \
             : ((G) == 16 ? FLEXSAE_DISPATCH_G(T, 16, kind, CALL) : FLEXSAE_DISPATCH_G(T, 8, kind, CALL)))
#define FLEXSAE_DISPATCH(wdt, G, kind, CALL)                                                       \
  ((wdt) == FLEXSAE_F32 ? FLEXSAE_DISPATCH_T(float, G, kind, CALL)                                 \
                        : ((wdt) == FLEXSAE_BF16 ? FLEXSAE_DISPATCH_T(__nv_bfloat16, G, kind, CALL) \
                                                 : FLEXSAE_DISPATCH_T(__half, G, kind, CALL)))

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace flexsae

using namespace flexsae;

extern "C" {

int flexsae_version(void) { return 200; }

const char* flexsae_last_error(void) { return t_err; }

int flexsae_last_launch_count(void) { return t_launches; }

int flexsae_set_option(const char* name, int64_t value) {
  if (!name) return fail(FLEXSAE_EINVAL, "option name is null");
  const bool lanes_ok = value == 0 || value == 8 || value == 16 || value == 32;
  if (!strcmp(name, "lanes_fwd") && lanes_ok) { g_opt.lanes_fwd = (int)value; return 0; }
  if (!strcmp(name, "lanes_bwd") && lanes_ok) { g_opt.lanes_bwd = (int)value; return 0; }
  if (!strcmp(name, "l2_budget_mb") && value >= 1 && value <= 4096) { g_opt.l2_budget_mb = (int)value; return 0; }
  if (!strcmp(name, "segments") && value >= 0 && value <= 256) { g_opt.segments = (int)value; return 0; }
  if (!strcmp(name, "pipeline") && (value == 0 || value == 1)) { g_opt.pipeline = (int)value; return 0; }
  if (!strcmp(name, "convert_offset_pct") && value >= 0 && value <= 100) { g_opt.convert_offset_pct = (int)value; return 0; }
  if (!strcmp(name, "direct_f32") && (value == 0 || value == 1)) { g_opt.direct_f32 = (int)value; return 0; }
  if (!strcmp(name, "exchange_blocks") && value >= 1 && value <= 4096) { g_opt.exchange_blocks = (int)value; return 0; }
  return fail(FLEXSAE_EINVAL, "unknown option or value: %s=%lld", name, (long long)value);
}

int64_t flexsae_get_option(const char* name) {
  if (!name) return -1;
  if (!strcmp(name, "lanes_fwd")) return g_opt.lanes_fwd;
  if (!strcmp(name, "lanes_bwd")) return g_opt.lanes_bwd;
  if (!strcmp(name, "l2_budget_mb")) return g_opt.l2_budget_mb;
  if (!strcmp(name, "segments")) return g_opt.segments;
  if (!strcmp(name, "pipeline")) return g_opt.pipeline;
  if (!strcmp(name, "convert_offset_pct")) return g_opt.convert_offset_pct;
  if (!strcmp(name, "direct_f32")) return g_opt.direct_f32;
  if (!strcmp(name, "exchange_blocks")) return g_opt.exchange_blocks;
  return -1;
}

int flexsae_choose_segments(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  return choose_segments(s, weight_dtype);
}

size_t flexsae_state_bytes(int kind, int64_t B, int64_t K, int64_t D, int segments) {
  if ((kind != FLEXSAE_TOPK && kind != FLEXSAE_HIER) || B < 1 || K < 1 || D < 1 || segments < 1) return 0;
  Shape s{B, K, 1, D};
  return state_floats(kind, s, segments) * sizeof(float);
}

size_t flexsae_fwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  return plan_fwd(s, weight_dtype).total;
}

size_t flexsae_bwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype, int dw_mode) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  if (dw_mode != FLEXSAE_DW_ATOMIC && dw_mode != FLEXSAE_DW_DETERMINISTIC) {
    fail(FLEXSAE_EINVAL, "unknown dweight mode %d", dw_mode);
    return 0;
  }
  return plan_bwd(s, weight_dtype, dw_mode).total;
}

int flexsae_loss_fwd(int kind, const int64_t* indices, const void* weight, const void* vals, const void* bias,
                     const void* target, float* loss_out, float* state_out, int segments, void* workspace,
                     size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                     int vals_dtype, int bias_dtype, int target_dtype, double inv_norm, int32_t* status, void* stream) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype) || !dtype_ok(target_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d, target %d)", vals_dtype, bias_dtype, target_dtype);
  int KS, NS;
  if (int rc = check_segments(kind, s, segments, &KS, &NS)) return rc;
  if (!indices || !weight || !vals || !bias || !target || !loss_out || !state_out || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(bias) || !aligned16(target) || !aligned16(state_out) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, bias, target, state and workspace must be 16-byte aligned");
  const FwdPlan p = plan_fwd(s, weight_dtype);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "forward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  FwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.bias = bias; a.target = target;
  a.loss_part = reinterpret_cast<float*>(workspace);
  a.state = state_out; a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype; a.bias_dtype = bias_dtype; a.target_dtype = target_dtype;
  a.KS = (kind == FLEXSAE_HIER) ? KS : round_up((int)K, kUnroll);
  a.NS = (kind == FLEXSAE_HIER) ? NS : 1;

#define CALL_FWD(T, G, H) launch_fwd<T, G, H>(a, p.pieces, st)
  cudaError_t e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_FWD);
#undef CALL_FWD
  if (e != cudaSuccess) return fail((int)e, "forward launch failed: %s", cudaGetErrorString(e));
  loss_finalize_kernel<<<1, 1024, 0, st>>>(a.loss_part, (size_t)p.pieces * B, inv_norm, loss_out);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "loss finalize launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"

namespace flexsae {
struct PeerInfo {  // batch-sharded call: who the other GPUs are and where their exchange buffers live
  int world, rank, seq_base;
  void* const* x;
  void* const* y;
  void* const* flags;
  void* mc_x;
  void* mc_y;
};

static int loss_bwd_impl(int kind, const int64_t* indices, const void* weight, const void* vals, const float* state,
                         int segments, const float* grad_out, void* dweight, void* dvals, void* dbias, void* workspace,
                         size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                         int vals_dtype, int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream,
                         const PeerInfo* peers) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d)", vals_dtype, bias_dtype);
  if (dw_mode != FLEXSAE_DW_ATOMIC && dw_mode != FLEXSAE_DW_DETERMINISTIC)
    return fail(FLEXSAE_EINVAL, "unknown dweight mode %d", dw_mode);
  int KS, NS;
  if (int rc = check_segments(kind, s, segments, &KS, &NS)) return rc;
  if (!indices || !weight || !vals || !state || !grad_out || !dweight || !dvals || !dbias || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(state) || !aligned16(dweight) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, state, dweight and workspace must be 16-byte aligned");
  const BwdPlan p = plan_bwd(s, weight_dtype, dw_mode);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "backward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* ws = reinterpret_cast<char*>(workspace);

  BwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.state = state; a.grad_out = grad_out;
  float* slabs[2] = {reinterpret_cast<float*>(ws + p.off_slab), reinterpret_cast<float*>(ws + p.off_slab + p.slab_bytes)};
  a.dweight = dweight;
  a.stage = nullptr;
  a.slot_of = nullptr;
  a.s0 = reinterpret_cast<float*>(ws + p.off_s0);
  a.dv_part = reinterpret_cast<float*>(ws + p.off_dv);
  a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype;
  a.scale = (float)(2.0 * inv_norm);
  a.KS = KS; a.NS = NS;
  a.slab_stride = p.PW;
  float* db_part = reinterpret_cast<float*>(ws + p.off_db);
  // An fp32 decoder needs no fp32 slab: dweight itself is the accumulation target (single GPU,
  // single-launch form).
  const bool direct = weight_dtype == FLEXSAE_F32 && dw_mode == FLEXSAE_DW_ATOMIC && !peers && g_opt.pipeline &&
                      g_opt.direct_f32;

  cudaError_t e = cudaSuccess;
  if (dw_mode == FLEXSAE_DW_DETERMINISTIC) {
    // Sort the (decoder row, position) pairs once; then per column piece: the same reverse walk,
    // but every contribution row is stored to its sorted slot, and the rows of each decoder row
    // are added in slot order straight into dweight.
    DetIndex ix;
    e = det_prepare(indices, B * K, F, ws + p.off_index, &ix, st, &t_launches);
    if (e != cudaSuccess) return fail((int)e, "sort launches failed: %s", cudaGetErrorString(e));
    a.stage = reinterpret_cast<float*>(ws + p.off_stage);
    a.slot_of = ix.slot_of;
    a.slab = a.conv_slab = nullptr;
    a.conv_piece = -1;
    float* part = reinterpret_cast<float*>(ws + p.off_part);
    for (int i = 0; i < p.pieces; i++) {
      a.piece = i;
#define CALL_DET(T, G, H) launch_bwd_det<T, G, H>(a, st)
      e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_DET);
#undef CALL_DET
      if (e != cudaSuccess) return fail((int)e, "backward launch failed: %s", cudaGetErrorString(e));
      e = det_reduce_piece(weight_dtype, p.G, a.stage, ix, (int)F, (int)D, i, part, dweight, st, &t_launches);
      if (e != cudaSuccess) return fail((int)e, "ordered sum launch failed: %s", cudaGetErrorString(e));
    }
  } else {
  // Both slabs are cleared once here; afterwards every conversion leaves its slab cleared.
  // Launch i accumulates piece i into slab i%2 and converts piece i-1 out of the other slab;
  // one more launch converts the last piece.
  if (direct) {
    e = cudaMemsetAsync(dweight, 0, (size_t)F * D * sizeof(float), st);
    a.slab_stride = (int)D;
  } else {
    e = cudaMemsetAsync(slabs[0], 0, 2 * p.slab_bytes, st);
  }
  if (e != cudaSuccess) return fail((int)e, "gradient clear failed: %s", cudaGetErrorString(e));
  if (peers) {
    int* counters = reinterpret_cast<int*>(ws + p.off_ctr);
    e = cudaMemsetAsync(counters, 0, (size_t)(3 * p.pieces + 6) * 4, st);
    if (e != cudaSuccess) return fail((int)e, "counter clear failed: %s", cudaGetErrorString(e));
    a.piece = a.conv_piece = -1;
    a.slab = a.conv_slab = nullptr;
    a.unit_blocks = a.conv_blocks = 0;
    a.conv_stride = 1;
    ShardArgs sa;
    sa.world = peers->world;
    sa.rank = peers->rank;
    sa.seq_base = peers->seq_base;
    sa.rows_per_rank = (int)((F + peers->world - 1) / peers->world);
    sa.mc_inbox = peers->mc_x;
    sa.mc_gathered = peers->mc_y;
    for (int r = 0; r < kMaxRanks; r++) {
      sa.inbox[r] = r < peers->world ? peers->x[r] : nullptr;
      sa.gathered[r] = r < peers->world ? peers->y[r] : nullptr;
      sa.flags_at[r] = r < peers->world ? reinterpret_cast<int*>(peers->flags[r]) : nullptr;
    }
#define CALL_SHARD(T, G, H) launch_bwd_sharded<T, G, H>(a, slabs[0], slabs[1], counters, p.pieces, sa, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_SHARD);
#undef CALL_SHARD
    if (e != cudaSuccess) return fail((int)e, "sharded backward launch failed: %s", cudaGetErrorString(e));
  } else if (g_opt.pipeline) {
    int* counters = reinterpret_cast<int*>(ws + p.off_ctr);
    e = cudaMemsetAsync(counters, 0, (size_t)(3 * p.pieces + 6) * 4, st);
    if (e != cudaSuccess) return fail((int)e, "counter clear failed: %s", cudaGetErrorString(e));
    a.piece = a.conv_piece = -1;
    a.slab = a.conv_slab = nullptr;
    a.unit_blocks = a.conv_blocks = 0;
    a.conv_stride = 1;
#define CALL_PIPE(T, G, H) launch_bwd_pipelined<T, G, H>(a, slabs[0], slabs[1], counters, p.pieces, direct, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_PIPE);
#undef CALL_PIPE
    if (e != cudaSuccess) return fail((int)e, "pipelined backward launch failed: %s", cudaGetErrorString(e));
  } else
  for (int i = 0; i <= p.pieces; i++) {
    a.piece = i < p.pieces ? i : -1;
    a.conv_piece = i - 1;
    a.slab = slabs[i & 1];
    a.conv_slab = slabs[(i & 1) ^ 1];
#define CALL_BWD(T, G, H) launch_bwd<T, G, H>(a, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_BWD);
#undef CALL_BWD
    if (e != cudaSuccess) return fail((int)e, "backward launch failed: %s", cudaGetErrorString(e));
  }
  }
  // dbias = coef * column sums of the final residual (TopK) or of the summed prefix residuals the
  // first-segment walkers left in s0 (Hierarchical): partial sums over row blocks, fixed order.
  const float* colsrc = kind == FLEXSAE_HIER ? a.s0 : state;
  column_sums_kernel<<<dim3((unsigned)((D + 127) / 128), p.row_blocks), 128, 0, st>>>(colsrc, (int)B, (int)D,
                                                                                      p.rows_per_block, db_part);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "column sums launch failed: %s", cudaGetErrorString(e));
  const size_t BK = (size_t)B * K;
  const int dv_blocks = (int)((BK + 255) / 256);
  const int db_blocks = (int)((D + 255) / 256);
  grads_finalize_kernel<<<dv_blocks + db_blocks, 256, 0, st>>>(a.dv_part, p.pieces, BK, dvals, vals_dtype, db_part,
                                                             p.row_blocks, (int)D, dbias, bias_dtype, dv_blocks,
                                                             grad_out, a.scale);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "gradient finalize launch failed: %s", cudaGetErrorString(e));
  return 0;
}
}  // namespace flexsae

extern "C" {

int flexsae_loss_bwd(int kind, const int64_t* indices, const void* weight, const void* vals, const float* state,
                     int segments, const float* grad_out, void* dweight, void* dvals, void* dbias, void* workspace,
                     size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                     int vals_dtype, int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream) {
  return loss_bwd_impl(kind, indices, weight, vals, state, segments, grad_out, dweight, dvals, dbias, workspace,
                       workspace_bytes, B, K, F, D, weight_dtype, vals_dtype, bias_dtype, inv_norm, dw_mode, status,
                       stream, nullptr);
}

int flexsae_shard_buffer_bytes(int64_t F, int64_t D, int weight_dtype, int world, size_t* x_bytes, size_t* y_bytes,
                               size_t* flag_bytes) {
  Shape s{1, 1, F, D};
  if (int rc = check_shape(FLEXSAE_HIER, s, weight_dtype)) return rc;
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (!x_bytes || !y_bytes || !flag_bytes) return fail(FLEXSAE_EINVAL, "null pointer argument");
  const BwdPlan p = plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC);
  const size_t rows_per_rank = (size_t)((F + world - 1) / world);
  *x_bytes = align_up(2 * (size_t)world * rows_per_rank * p.PW * dtype_size(weight_dtype), 256);  // inbox
  *y_bytes = *x_bytes;                                                                           // gather buffer
  *flag_bytes = 256;
  return 0;
}

int flexsae_loss_bwd_sharded(int kind, const int64_t* indices, const void* weight, const void* vals,
                             const float* state, int segments, const float* grad_out, void* dweight, void* dvals,
                             void* dbias, void* workspace, size_t workspace_bytes, int64_t B, int64_t K, int64_t F,
                             int64_t D, int weight_dtype, int vals_dtype, int bias_dtype, double inv_norm,
                             int32_t* status, void* stream, int world, int rank, int seq_base, void* const* x_ptrs,
                             void* const* y_ptrs, void* const* flag_ptrs, void* multicast_x, void* multicast_y) {
  if (world < 2 || world > kMaxRanks) return fail(FLEXSAE_EINVAL, "world size %d outside [2, %d]", world, kMaxRanks);
  if (rank < 0 || rank >= world) return fail(FLEXSAE_EINVAL, "rank %d outside [0, %d)", rank, world);
  if (!x_ptrs || !y_ptrs || !flag_ptrs) return fail(FLEXSAE_EINVAL, "null pointer argument");
  for (int r = 0; r < world; r++)
    if (!x_ptrs[r] || !y_ptrs[r] || !flag_ptrs[r] || !aligned16(x_ptrs[r]) || !aligned16(y_ptrs[r]))
      return fail(FLEXSAE_EINVAL, "exchange buffer of rank %d is null or not 16-byte aligned", r);
  if (seq_base < 1) return fail(FLEXSAE_EINVAL, "seq_base must be >= 1");
  if ((multicast_x == nullptr) != (multicast_y == nullptr) || !aligned16(multicast_x) || !aligned16(multicast_y))
    return fail(FLEXSAE_EINVAL, "multicast addresses must both be given (16-byte aligned) or both be NULL");
  PeerInfo peers{world, rank, seq_base, x_ptrs, y_ptrs, flag_ptrs, multicast_x, multicast_y};
  return loss_bwd_impl(kind, indices, weight, vals, state, segments, grad_out, dweight, dvals, dbias, workspace,
                       workspace_bytes, B, K, F, D, weight_dtype, vals_dtype, bias_dtype, inv_norm, FLEXSAE_DW_ATOMIC,
                       status, stream, &peers);
}

int flexsae_shard_slots(int64_t F, int64_t D, int weight_dtype) {
  Shape s{1, 1, F, D};
  if (check_shape(FLEXSAE_HIER, s, weight_dtype)) return 0;
  return plan_bwd(s, weight_dtype, FLEXSAE_DW_ATOMIC).pieces + 3;
}

// ---- forward for callers that cannot provide scratch memory ------------------------------------
// The per-(piece, row) partial losses of the forward normally live in caller memory.  Here they
// live in a fixed array inside the library image: every GPU that loads the library carries these
// bytes until the process exits.
#define FLEXSAE_STATIC_PARTIALS (1u << 18) /* floats: 1 MiB */
static __device__ __align__(256) float g_static_loss_partials[FLEXSAE_STATIC_PARTIALS];

static std::mutex g_static_mutex;
static float* g_static_partials_addr[64];  // device ordinal -> device address of the array above

int flexsae_loss_fwd_static_scratch(int kind, const int64_t* indices, const void* weight, const void* vals,
                                    const void* bias, const void* target, float* loss_out, float* state_out,
                                    int segments, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                                    int vals_dtype, int bias_dtype, int target_dtype, double inv_norm,
                                    int32_t* status, void* stream) {
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  const size_t need = plan_fwd(s, weight_dtype).total;
  const size_t have = sizeof(float) * FLEXSAE_STATIC_PARTIALS;
  if (need > have)
    return fail(FLEXSAE_EUNSUPPORTED,
                "the built-in scratch holds %zu bytes but this shape needs %zu (column pieces x B = %lld partial "
                "sums; at most %u): use flexsae_loss_fwd with caller memory",
                have, need, (long long)(need / sizeof(float)), (unsigned)FLEXSAE_STATIC_PARTIALS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(FLEXSAE_EUNSUPPORTED, "device ordinal %d outside [0, 64)", dev);
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_partials_addr[dev]) {
      // In host code the array's name is only a handle; the address the kernels need is asked
      // from the runtime once per device, with that device current.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_loss_partials);
      if (e != cudaSuccess) return fail((int)e, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      g_static_partials_addr[dev] = reinterpret_cast<float*>(p);
    }
    scratch = g_static_partials_addr[dev];
  }
  // Every partial the final sum reads is written by this call's forward kernel first, so nothing
  // left over from an earlier call is ever read and nothing needs clearing.
  return flexsae_loss_fwd(kind, indices, weight, vals, bias, target, loss_out, state_out, segments, scratch, have, B, K,
                          F, D, weight_dtype, vals_dtype, bias_dtype, target_dtype, inv_norm, status, stream);
}

}  // extern "C"
