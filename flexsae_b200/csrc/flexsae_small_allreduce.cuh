// Sum of a short vector (the scalar loss, dbias) over the GPUs of one node, over peer memory: one
// block, one launch, a few microseconds -- the sharded losses need two such sums per step and a
// library all-reduce costs more in latency than the payload is worth.
#pragma once

#include "flexsae_sharded.cuh"

namespace flexsae {

constexpr int kSmallThreads = 1024;
constexpr int kSmallFlagBytes = 256;  // the first bytes of every rank's buffer: one int per sender

struct SmallReduceArgs {
  const void* in;  // n values of `dtype` (may be the same memory as out)
  void* out;
  int n, dtype, world, rank, seq;
  long long capacity;  // floats per (parity, sender) cell of the exchange buffer
  long long wait_ns;   // how long the wait for the other ranks may last
  int32_t* status;
  void* buf[kMaxRanks];  // rank o's buffer: flags, then float data[2][world][capacity]
};

// Every rank pushes its values (as fp32) into cell [seq & 1][rank] of every rank's buffer, then
// announces `seq` in every rank's flag array; when all senders have announced, the cells are added
// in rank order, so every rank gets the same bits.  Two cells per sender suffice: a rank can only
// be one call ahead of the slowest one, because call seq+1 does not complete anywhere before every
// rank has at least started it, i.e. finished reading call seq (calls on one rank are stream-ordered).
__global__ void __launch_bounds__(kSmallThreads) small_allreduce_kernel(const SmallReduceArgs a) {
  const int par = a.seq & 1;
  const size_t cell = ((size_t)par * a.world + a.rank) * a.capacity;
  for (int i = threadIdx.x; i < a.n; i += kSmallThreads) {
    const float v = load_scalar(a.in, a.dtype, i);
    for (int o = 0; o < a.world; o++)
      reinterpret_cast<float*>(reinterpret_cast<char*>(a.buf[o]) + kSmallFlagBytes)[cell + i] = v;  // peer store
  }
  __syncthreads();
  if ((int)threadIdx.x < a.world)  // the release orders every store this block made before the flag
    st_release_sys(reinterpret_cast<int*>(a.buf[threadIdx.x]) + a.rank, a.seq);
  if ((int)threadIdx.x < a.world) {
    const int* flag = reinterpret_cast<const int*>(a.buf[a.rank]) + threadIdx.x;
    BoundedWait bw;
    while (ld_acquire_sys(flag) - a.seq < 0) {
      __nanosleep(100);
      if (bw.give_up(a.status, a.wait_ns)) break;
    }
  }
  __syncthreads();
  const float* mine = reinterpret_cast<const float*>(reinterpret_cast<const char*>(a.buf[a.rank]) + kSmallFlagBytes) +
                      (size_t)par * a.world * a.capacity;
  for (int i = threadIdx.x; i < a.n; i += kSmallThreads) {
    float s = 0.f;
    for (int r = 0; r < a.world; r++) s += __ldcg(mine + (size_t)r * a.capacity + i);
    store_scalar(a.out, a.dtype, i, s);
  }
}

}  // namespace flexsae
