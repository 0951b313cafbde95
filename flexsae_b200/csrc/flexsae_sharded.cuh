// Batch-sharded backward: the single-launch pipeline with the cross-GPU sum of dweight done by its
// own blocks over NVLink peer memory.
#pragma once

#include "flexsae_backward.cuh"

namespace flexsae {

// ---- batch-sharded backward: pipelined kernel + dweight reduction over peer memory ----------------
// Every rank (one GPU each, same node) runs this kernel on its own batch shard.  The converting
// blocks of the single-launch pipeline do the cross-GPU sum of dweight themselves, piece by piece,
// overlapped with the accumulation of the following pieces.  All traffic between GPUs is posted
// STORES into the peers' buffers (a remote load would stall its thread for microseconds; a store
// does not), all loads are local.  With L = conv_lag, slot p
//   accumulates piece p (unit blocks) into slab p % nslabs,
//   converts the local slab of piece p-L (decoder dtype) and SCATTERS it: every decoder row goes to
//     the inbox of the rank that owns that row block (reduce-scatter by push),
//   reduces piece p-L-1: this rank sums the N inbox copies of ITS row block (fixed rank order, fp32),
//     writes its own dweight rows and BROADCASTS the reduced rows into every peer's gather buffer,
//   copies piece p-L-2: the other ranks' reduced row blocks from the local gather buffer to dweight.
// Two flags per (rank, peer) carry all cross-GPU ordering.  When the last converting block of slot p
// finishes, the rank publishes seq_base + p in its SCATTER flag on every rank; when the last exchange
// block of slot p finishes, the same in its EXCHANGE flag.  Who waits for what:
//   converting blocks of slot p (they overwrite the inbox half that the reduce of slot p-1 read):
//     every rank's exchange flag >= slot p-1;
//   exchange blocks of slot p: every rank's scatter flag >= slot p-1 (the inbox copies of the piece
//     they reduce are complete) and, because the gather buffer is double-buffered as well, every
//     rank's exchange flag >= slot p-1 (the previous piece has been broadcast, the one before copied).
// A rank publishes its flags strictly in slot order (the last block of slot p first waits for the
// rank's own flag of slot p-1), so a flag value really means "all slots up to this one".
// With peer-mapped dweight tables there is no gather buffer and the exchange blocks wait for the
// scatter flags only (plus, in the very last slot, for every rank's last broadcast): an exchange may
// then take longer than one slot without holding anything up.  Waits are bounded like the local
// ones.  Plain peer stores only: no multicast of any kind.
constexpr int kMaxRanks = 8;
constexpr int kScatterFlags = 32;  // offset (ints) of the scatter flags inside a rank's flag array
struct ShardArgs {
  PipeArgs p;
  int* slot_done;  // [pieces + 3] exchange blocks of a slot that have finished
  int* scatter_done;  // [pieces + 3] converting blocks of a slot whose peer stores are out
  int world, rank, rows_per_rank, seq_base;
  int exch_blocks;  // blocks per slot that reduce / broadcast / copy older pieces
  int exch_offset;  // unit blocks of a slot dispatched before its exchange blocks (<= conv_offset)
  int rotate;       // 1: each rank starts its scatter sweep at its right-hand neighbour's row block
  int fan_out;      // 1: the flags of a finished slot are stored by one thread per destination rank
  void* mc_inbox;     // multicast address of the inbox region of ALL ranks (NULL: plain peer stores)
  void* mc_gathered;  // multicast address of the gather buffers of all ranks
  void* inbox[kMaxRanks];    // rank o's inbox: [2][world][rows_per_rank][PW]
  void* gathered[kMaxRanks]; // rank o's gather buffer: [2][world * rows_per_rank][PW]
  int* flags_at[kMaxRanks];  // flag array living on rank s: [r] = last slot whose exchange rank r finished,
                             // [kScatterFlags + r] = last slot whose scatter rank r finished
  void* dweight_at[kMaxRanks];  // every rank's dweight when those are peer-mapped: the broadcast then
                                // lands in place and the gather buffer and its copy are not used (else NULL)
};

// Tuning builds (-DFLEXSAE_TRACE) record, per slot, when each block role started and ended on
// this GPU's nanosecond timer; flexsae_debug_trace_read returns the table.  Minima are kept as
// the maximum of the complement so that a cleared table is all zeros.
enum { kTrUnitStart, kTrUnitEnd, kTrConvEntry, kTrConvStart, kTrConvEnd, kTrExchEntry, kTrExchStart, kTrExchEnd, kTrFields };
#ifdef FLEXSAE_TRACE
__device__ unsigned long long g_trace[64][kTrFields];
__device__ __forceinline__ void trace_mark(int slot, int field, bool is_min) {
  if (threadIdx.x == 0 && slot < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(&g_trace[slot][field], is_min ? ~t : t);
  }
}
#define FLEXSAE_TRACE_MIN(slot, field) trace_mark(slot, field, true)
#define FLEXSAE_TRACE_MAX(slot, field) trace_mark(slot, field, false)
#else
#define FLEXSAE_TRACE_MIN(slot, field)
#define FLEXSAE_TRACE_MAX(slot, field)
#endif

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// flag = max(flag, v) with release semantics: a posted update that can never move a flag backwards,
// whatever order the updates of different publishers arrive in
__device__ __forceinline__ void red_max_release_sys(int* p, int v) {
  asm volatile("red.release.sys.global.max.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One thread per (rank, flag kind) polls: lanes 0..world-1 of warp 0 the exchange flags, of warp 1
// the scatter flags (this rank's own flags too: its own earlier slots use the same buffers).
__device__ __forceinline__ void wait_peers(const ShardArgs& sa, bool need_exchange, int exchange_target,
                                           bool need_scatter, int scatter_target) {
  const int kind = threadIdx.x >> 5, s = threadIdx.x & 31;
  if (kind < 2 && s < sa.world && (kind == 0 ? need_exchange : need_scatter)) {
    int32_t* status = sa.p.b.status;
    const int* flag = sa.flags_at[sa.rank] + kind * kScatterFlags + s;
    const int target = kind == 0 ? exchange_target : scatter_target;
    BoundedWait bw;
    while (ld_acquire_sys(flag) - target < 0) {  // difference: robust to wrap-around
      __nanosleep(100);
      if (bw.give_up(status, sa.p.wait_ns)) break;
    }
  }
  __syncthreads();
}

// local slab (fp32, permuted columns) -> decoder dtype, natural column order, each decoder row
// stored into the inbox of the rank owning its row block; clears the slab
// ROTATE: the sweep over the slab is cut into chunks of one grid stride (a few thousand decoder rows)
// and every rank starts at a different chunk, so that at any moment the ranks store to different
// owners instead of all to one.  Only the chunk order changes -- the per-item arithmetic is that of
// the plain sweep: an earlier form that rotated every item index separately made this loop, and
// with it every slot of the pipeline, 25 % slower even with the rotation switched off.
template <typename T, int G, bool ROTATE>
__device__ __forceinline__ void slab_scatter(float* slab, const ShardArgs& sa, int piece, int cta, int nctas) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int IL = FLEXSAE_CONVERT_IL;
  const int F = sa.p.b.F;
  const int rpr = sa.rows_per_rank;
  const size_t total = (size_t)F * G;  // 16-byte items of the piece
  const size_t stride = (size_t)nctas * kThreads;
  const size_t slot_off = ((size_t)(piece & 1) * sa.world + sa.rank) * rpr * PW;  // [parity][sender = me]
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const int n_chunks = (int)((total + stride - 1) / stride);
  const int shift = ROTATE ? (int)((long long)n_chunks * ((sa.rank + 1) % sa.world) / sa.world) : 0;
  const size_t first = (size_t)cta * kThreads + threadIdx.x;
  // item handled as number q of the group of IL chunks that starts at chunk c0 (>= total: none)
  auto item_at = [&](int c0, int q) -> size_t {
    int c = c0 + q;
    if (c >= n_chunks) return total;
    if (ROTATE) {
      c += shift;
      if (c >= n_chunks) c -= n_chunks;
    }
    return (size_t)c * stride + first;
  };
  for (int c0 = 0; c0 < n_chunks; c0 += IL) {
    float4 lo[IL], hi[IL];
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = item_at(c0, q);
      if (i < total) {
        float* sp = slab + (i / G) * PW + (i % G) * 4;
        lo[q] = __ldcg(reinterpret_cast<const float4*>(sp));
        if (VEC == 8) hi[q] = __ldcg(reinterpret_cast<const float4*>(sp + G * 4));
      }
    }
#pragma unroll
    for (int q = 0; q < IL; q++) {
      const size_t i = item_at(c0, q);
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
// and every peer's gather buffer (IN_PLACE: straight into every peer's dweight rows instead).
// IL items per thread in flight (IL * world local 16-byte loads).
template <typename T, int G, int IL, bool IN_PLACE>
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
        const int col = piece * PW + (int)(i % G) * VEC;
        const size_t dw_off = (size_t)(row0 + i / G) * D + col;
        if (IN_PLACE) {
#pragma unroll
          for (int o = 0; o < kMaxRanks; o++)
            if (o < sa.world && o != sa.rank && col < D)
              *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.dweight_at[o]) + dw_off) = out;  // peer store
        } else {
#pragma unroll
          for (int o = 0; o < kMaxRanks; o++)
            if (o < sa.world && o != sa.rank)
              *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.gathered[o]) + gat_off + i * VEC) = out;  // peer store
        }
        if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(sa.p.b.dweight) + dw_off) = out;
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

// One more block of a slot has finished its scatter (`scatter`) or exchange work: count it, and if
// it was the last of `target`, publish `seq_base + slot` in this rank's flag of that kind on every
// rank.  All threads of the block call it.
//  * A flag says "everything up to this slot", so it may only move forward in slot order: the blocks
//    of one slot can finish before those of the previous one (nothing else orders them), and then
//    this rank's flag of the previous slot -- written by the last block of that slot -- has to go
//    out first (`first` = there is no previous slot of this kind in this call).
//  * The rank's own copy is stored FIRST, so that its own waiting blocks and the next slot's
//    publisher go on without an NVLink round trip; the peers' copies are updated with a posted
//    atomic max, so that the updates of consecutive slots, issued by different blocks, may arrive in
//    any order without a flag ever falling back.  (Publishing the peers first and the own copy last
//    with plain stores is also correct but put two NVLink round trips into every slot's critical
//    path: measured +0.17 ms per step on two GPUs.)
__device__ __forceinline__ void count_and_publish(const ShardArgs& sa, bool scatter, int* counter, int target, int slot,
                                                  bool first) {
  const int kind_off = scatter ? kScatterFlags : 0;
  int publish = 0;  // decided by thread 0, handed to the block through the barrier's vote (no shared variable)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // this block's peer stores and dweight writes before the count moves
    const int old = atomicAdd(counter, 1);
    const bool last = old == target - 1;
    if (last) __threadfence_system();  // acquire side: what the other blocks did before THEIR count moved
    if (last && !first) {
      const int* own = sa.flags_at[sa.rank] + kind_off + sa.rank;
      BoundedWait bw;
      while (ld_acquire_sys(own) - (sa.seq_base + slot - 1) < 0) {
        __nanosleep(100);
        if (bw.give_up(sa.p.b.status, sa.p.wait_ns)) break;
      }
    }
    if (last) st_release_sys(sa.flags_at[sa.rank] + kind_off + sa.rank, sa.seq_base + slot);
    publish = last;
  }
  if (__syncthreads_or(publish)) {  // uniform over the block
    const int value = sa.seq_base + slot;
    if (sa.fan_out) {  // one thread per destination: the updates travel side by side
      if ((int)threadIdx.x < sa.world && (int)threadIdx.x != sa.rank)
        red_max_release_sys(sa.flags_at[threadIdx.x] + kind_off + sa.rank, value);
    } else if (threadIdx.x == 0) {
      for (int s = 0; s < sa.world; s++)
        if (s != sa.rank) red_max_release_sys(sa.flags_at[s] + kind_off + sa.rank, value);
    }
  }
}

// Exchange work of slot p (all threads of an exchange block): wait for what it reads to be
// complete, reduce + broadcast piece p-2, copy piece p-3 out of the gather buffer.
template <typename T, int G>
__device__ __forceinline__ void exchange_slot(const ShardArgs& sa, int p, int exch_idx, int exch_n, bool in_place) {
  const int P = sa.p.pieces, L = sa.p.conv_lag;
  const int reduce_piece = p - L - 1, copy_piece = p - L - 2;
  const int last_slot = P + L + 1, last_scatter_slot = P + L - 1;
  FLEXSAE_TRACE_MIN(p, kTrExchEntry);
  // the inbox copies of the piece to reduce are complete (scattered in slot p-1); through the gather
  // buffer also: the previous piece has arrived in it and the one before has been copied out everywhere;
  // in place: the very last slot returns only when every rank's last broadcast has landed here
  if (p >= 2) wait_peers(sa, !in_place || p == last_slot, sa.seq_base + p - 1, true, sa.seq_base + min(p - 1, last_scatter_slot));
  FLEXSAE_TRACE_MIN(p, kTrExchStart);
  if (reduce_piece >= 0 && reduce_piece < P && sa.mc_inbox) {
    switch_reduce_broadcast<T, G>(sa, reduce_piece, exch_idx, exch_n);
  } else if (reduce_piece >= 0 && reduce_piece < P) {
    if (in_place) {
      if (sa.world <= 2) reduce_broadcast<T, G, 4, true>(sa, reduce_piece, exch_idx, exch_n);
      else if (sa.world <= 4) reduce_broadcast<T, G, 2, true>(sa, reduce_piece, exch_idx, exch_n);
      else reduce_broadcast<T, G, 1, true>(sa, reduce_piece, exch_idx, exch_n);
    } else {
      if (sa.world <= 2) reduce_broadcast<T, G, 4, false>(sa, reduce_piece, exch_idx, exch_n);
      else if (sa.world <= 4) reduce_broadcast<T, G, 2, false>(sa, reduce_piece, exch_idx, exch_n);
      else reduce_broadcast<T, G, 1, false>(sa, reduce_piece, exch_idx, exch_n);
    }
  }
  // in-place broadcast: nothing to copy, but the last slot still waits (above) until every rank's
  // last broadcast has landed in this rank's dweight
  if (copy_piece >= 0 && copy_piece < P && !in_place) copy_gathered<T, G>(sa, copy_piece, exch_idx, exch_n);
}

// Block roles inside slot p of the sharded launch (slots 0 .. pieces + conv_lag + 1):
//   exchange blocks (sa.exch_blocks, after the first sa.exch_offset unit blocks): reduce + broadcast
//     and copy of older pieces -- local loads and posted stores only, so a few blocks keep up;
//   unit blocks: accumulate piece p;
//   converting blocks (inserted at conv_offset): slab of piece p - conv_lag -> scattered to the owners, cleared.
// The conv_lag + 2 draining slots after the last piece have no unit blocks; their blocks are exchange
// blocks, except that the first conv_lag of them still hold the converting blocks of the last pieces.
template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(kThreads, FLEXSAE_BWD_MINB) decoder_loss_bwd_sharded_kernel(const ShardArgs sa) {
  extern __shared__ __align__(128) uint4 smem[];
  const PipeArgs& pa = sa.p;
  const int P = pa.pieces, L = pa.conv_lag;
  const int E = sa.exch_blocks;
  const int per = E + pa.unit_blocks + pa.conv_blocks;
  const int body = P * per;
  int p, exch_idx = -1, conv_idx = -1, unit_block = -1;
  int exch_n = E;  // blocks that share the exchange work of this slot
  const bool in_place = sa.dweight_at[0] != nullptr && sa.mc_inbox == nullptr;
  const int bid = role_index(pa.ticket, smem);
  if (bid >= body) {  // draining slots: no unit blocks
    const int t = bid - body;
    const int dper = E + pa.conv_blocks;
    p = P + t / dper;
    const int r = t - (p - P) * dper;
    if (p < P + L && r >= E) {
      conv_idx = r - E;  // the last conv_lag slabs are still to be converted
    } else {
      exch_idx = r;
      exch_n = (p < P + L) ? E : dper;  // afterwards every block helps with the exchange
    }
  } else {
    p = bid / per;
    int r = bid - p * per;
    if (r < sa.exch_offset) {
      unit_block = r;
    } else if (r < sa.exch_offset + E) {
      exch_idx = r - sa.exch_offset;
    } else {
      r -= E;
      if (r >= pa.conv_offset && r < pa.conv_offset + pa.conv_blocks) conv_idx = r - pa.conv_offset;
      else unit_block = r < pa.conv_offset ? r : r - pa.conv_blocks;
    }
  }
  if (unit_block >= 0) {
    // this slab last held piece p - nslabs, which the converting blocks of slot p - nslabs + L cleared
    if (p >= pa.nslabs) wait_count(pa.conv_done + (p - pa.nslabs + L), pa.conv_blocks, pa.b.status, pa.wait_ns);
    FLEXSAE_TRACE_MIN(p, kTrUnitStart);
    walk_units<T, G, HIER, false>(pa.b, unit_block, p, pa.slabs[p % pa.nslabs], smem);
    signal_done(pa.walk_done + p);
    FLEXSAE_TRACE_MAX(p, kTrUnitEnd);
    return;
  }
  if (conv_idx >= 0) {
    FLEXSAE_TRACE_MIN(p, kTrConvEntry);
    const int q = p - L;
    if (q >= 0 && q < P) {
      wait_count(pa.walk_done + q, pa.unit_blocks, pa.b.status, pa.wait_ns);  // the local slab is complete
      wait_peers(sa, true, sa.seq_base + p - 1, false, 0);  // the owners have reduced what this half of their inbox held
      FLEXSAE_TRACE_MIN(p, kTrConvStart);
      if (sa.mc_inbox) slab_to_own_copy<T, G>(pa.slabs[q % pa.nslabs], sa, q, conv_idx, pa.conv_blocks);
      else if (sa.rotate) slab_scatter<T, G, true>(pa.slabs[q % pa.nslabs], sa, q, conv_idx, pa.conv_blocks);
      else slab_scatter<T, G, false>(pa.slabs[q % pa.nslabs], sa, q, conv_idx, pa.conv_blocks);
    }
    signal_done(pa.conv_done + p);
    FLEXSAE_TRACE_MAX(p, kTrConvEnd);
  } else {
    exchange_slot<T, G>(sa, p, exch_idx, exch_n, in_place);
  }
  __syncthreads();
  if (exch_idx >= 0) { FLEXSAE_TRACE_MAX(p, kTrExchEnd); }
  const bool scatter = conv_idx >= 0;
  // slot 0 has no earlier slot of this launch to publish behind (the previous launch on this rank has
  // completed, flags included: launches of one rank are stream-ordered)
  count_and_publish(sa, scatter, (scatter ? sa.scatter_done : sa.slot_done) + p, scatter ? pa.conv_blocks : exch_n, p, p == 0);
}

}  // namespace flexsae
