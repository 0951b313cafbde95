// Backward kernels of the fused decoder losses: the reverse walk with L2-resident fp32 slabs, the
// single-launch pipeline over all column pieces, and the small finalising kernels.
#pragma once

#include "flexsae_kernel_args.cuh"

namespace flexsae {

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
  // The kernels declare `smem` 128-byte aligned: a quarter-warp's 8 x 16 bytes then sit in one
  // 128-byte line whatever static shared memory a kernel also has (an offset of 16 bytes made every
  // ring access straddle two lines and cost 7 % of the backward's time).
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
  extern __shared__ __align__(128) uint4 smem[];  // ring, staged pairs [UPC][KS], then (deterministic mode) int slots[UPC][KS]
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
// All column pieces in ONE grid, ordered slot by slot.  Slot p holds the unit blocks of piece p and,
// inserted part-way, the blocks that convert piece p - conv_lag.  The fp32 slabs rotate: piece p
// accumulates into slab p % nslabs.  Two counters per piece carry the only dependencies:
//   converting blocks of piece q wait until all unit blocks of piece q have finished;
//   unit blocks of piece p wait until piece p - nslabs (same slab) has been converted and cleared.
// A unit block runs for about as long as a whole slot lasts, so the last unit blocks of piece q end
// most of a slot after the first blocks of piece q+1 started; only then can piece q be converted, and
// with two slabs piece q+2 had to wait for exactly that conversion: the chain walk -> convert -> walk
// set the pace (70 us per piece at the headline shape against 51 us of work).  With three slabs and a
// lag of two the conversion of piece q runs a slot later, finds its walk long finished, and has a whole
// slot before anybody needs the slab back.
// Every wait is on blocks with LOWER role indices, which start first (see role_index), so the
// lowest unfinished block never waits on anything unfinished.  Waits are bounded in time (see
// BoundedWait): a block that gives up sets FLEXSAE_STATUS_PIPELINE_TIMEOUT and carries on (the
// result is then invalid but the GPU is not held).
constexpr int kMaxSlabs = 4;
struct PipeArgs {
  BwdArgs b;
  float* slabs[kMaxSlabs];
  int nslabs;    // fp32 slabs in rotation: piece p accumulates into slab p % nslabs
  int conv_lag;  // the converting blocks of slot p convert piece p - conv_lag (1 <= conv_lag < nslabs)
  int* walk_done;  // [pieces]
  int* conv_done;  // [pieces] (sharded kernel: per slot)
  int pieces, unit_blocks, conv_blocks, conv_offset;
  int* ticket;  // NULL: blocks take their roles by blockIdx.x; else by the order in which they start
  long long wait_ns;  // how long one wait may last before the block gives up (option "wait_limit_ms")
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  // an acquire load on purpose: a relaxed one may be served from a stale L1 line and see the
  // counter move late (measured: +0.7 ms per step with relaxed polling and one fence afterwards)
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The bound of every polling loop in this library, in wall-clock time on the GPU's nanosecond
// timer (a poll count would make the limit depend on clock speed and on how long a poll takes
// across NVLink).  Every 64th poll looks at the timer and at the status word; the first look
// sets the deadline.  give_up() answers true when the deadline has passed or when another block
// has already given up (then nobody waits any more and the launch drains quickly), and records
// FLEXSAE_STATUS_PIPELINE_TIMEOUT.
struct BoundedWait {
  unsigned long long deadline = 0;
  int polls = 0;
  __device__ __forceinline__ bool give_up(int32_t* status, long long limit_ns) {
    if ((++polls & 63) != 0) return false;
    const unsigned long long now = global_ns();
    if (deadline == 0) {
      deadline = now + (unsigned long long)limit_ns;
      return false;
    }
    const bool abandoned = status && (*reinterpret_cast<volatile int32_t*>(status) & FLEXSAE_STATUS_PIPELINE_TIMEOUT);
    if (now > deadline || abandoned) {
      if (status) atomicOr(status, FLEXSAE_STATUS_PIPELINE_TIMEOUT);
      return true;
    }
    return false;
  }
};

__device__ __forceinline__ void wait_count(const int* ctr, int target, int32_t* status, long long wait_ns) {
  if (threadIdx.x == 0) {
    BoundedWait bw;
    while (ld_acquire(ctr) < target) {
      __nanosleep(200);
      if (bw.give_up(status, wait_ns)) break;
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

// The waits of the single-launch kernels are safe as long as a block never starts before the blocks
// it waits for.  Hardware hands out blockIdx.x in increasing order in practice, but nothing
// documents that; with a ticket counter the role index IS the starting order, by construction.
__device__ __forceinline__ int role_index(int* ticket, uint4* smem) {
  if (!ticket) return (int)blockIdx.x;
  int* word = reinterpret_cast<int*>(smem);  // the dynamic shared memory is not in use yet
  if (threadIdx.x == 0) *word = atomicAdd(ticket, 1);
  __syncthreads();
  const int mine = *word;
  __syncthreads();
  return mine;
}

template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(kThreads, FLEXSAE_BWD_MINB) decoder_loss_bwd_pipelined_kernel(const PipeArgs pa) {
  extern __shared__ __align__(128) uint4 smem[];
  const int bid = role_index(pa.ticket, smem);
  const int per = pa.unit_blocks + pa.conv_blocks;
  const int body = pa.pieces * per;
  int p, conv_idx = -1, unit_block = -1;
  if (bid >= body) {  // conv_lag trailing slots: only converting blocks, for the last pieces
    const int t = bid - body;
    p = pa.pieces + t / pa.conv_blocks;
    conv_idx = t - (p - pa.pieces) * pa.conv_blocks;
  } else {
    p = bid / per;
    const int r = bid - p * per;
    if (r >= pa.conv_offset && r < pa.conv_offset + pa.conv_blocks) conv_idx = r - pa.conv_offset;
    else unit_block = r < pa.conv_offset ? r : r - pa.conv_blocks;
  }
  if (conv_idx >= 0) {
    const int q = p - pa.conv_lag;
    if (q < 0) return;
    wait_count(pa.walk_done + q, pa.unit_blocks, pa.b.status, pa.wait_ns);
    convert_slab<T, G, true>(pa.slabs[q % pa.nslabs], pa.b.dweight, pa.b.F, pa.b.D, q, conv_idx, pa.conv_blocks);
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
  if (p >= pa.nslabs) wait_count(pa.conv_done + (p - pa.nslabs), pa.conv_blocks, pa.b.status, pa.wait_ns);
  walk_units<T, G, HIER, false>(pa.b, unit_block, p, pa.slabs[p % pa.nslabs], smem);
  signal_done(pa.walk_done + p);
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

}  // namespace flexsae
