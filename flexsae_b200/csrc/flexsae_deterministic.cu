// Deterministic dweight: stable sort of the (decoder row, position) pairs and fixed-order
// segmented sums of staged contributions.
//
// The reference's TopK backward groups positions by decoder row with a counting sort whose
// placement uses fetch-add (torch-ext/flex_sae/topk_kernels.py:71-94), so the order inside a
// row's segment -- and with it the float sum -- changes from run to run, and its Hierarchical
// backward adds with float atomics (hierarchical_kernels.py:155-161).  Here the order is total:
// pairs are sorted by (decoder row, position b*K+k) with a stable LSD radix sort, every pair's
// contribution row is written to its sorted slot, and each decoder row's slots are added strictly
// in slot order.  Long segments (skewed indices) are cut into 32-slot items whose partial rows
// are then added in item order, so the result is still one fixed parenthesisation.
#include "flexsae_deterministic.cuh"

namespace flexsae {

static constexpr int kSortTile = 1024;   // keys per CTA in the histogram / scatter passes (one warp walks a tile in order)
static constexpr int kItemSlots = 32;    // sorted slots per first-level item

// ---- stable LSD radix sort of (key = decoder row, value = position) -----------------------------
template <bool FIRST>
__global__ void __launch_bounds__(256) sort_hist_kernel(const int64_t* __restrict__ indices, const int* __restrict__ keys, int n,
                                                        int F, int shift, int radix, int ntiles, int* __restrict__ counts) {
  extern __shared__ int hist[];
  for (int i = threadIdx.x; i < radix; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  const int t0 = blockIdx.x * kSortTile;
  const int t1 = min(n, t0 + kSortTile);
  for (int i = t0 + threadIdx.x; i < t1; i += blockDim.x) {
    int k;
    if (FIRST) {
      int64_t x = indices[i];
      k = ((uint64_t)x >= (uint64_t)F) ? 0 : (int)x;  // same clamp as the loss kernels
    } else {
      k = keys[i];
    }
    atomicAdd(&hist[(k >> shift) & (radix - 1)], 1);  // integer counts: order-independent
  }
  __syncthreads();
  for (int d = threadIdx.x; d < radix; d += blockDim.x) counts[(size_t)d * ntiles + blockIdx.x] = hist[d];
}

// ---- in-place exclusive scan of n ints ----------------------------------------------------------
// Blocks of 4096 ints: per-block sums, a scan of those sums by one CTA, then every block scans
// itself and adds its offset.  (One CTA walking the whole array took 170 us for the 131072
// digit counts of the headline shape, six times per backward.)
static constexpr int kScanBlock = 4096;  // 1024 threads x int4

// exclusive scan of up to 4096 ints held as one int4 per thread; returns the four outputs and the block total
__device__ __forceinline__ int4 scan_block(int4 v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = v.x + v.y + v.z + v.w;
  int incl = s;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += up;
    }
    warp_sums[lane] = w;  // inclusive totals of the warps
  }
  __syncthreads();
  const int before = (warp ? warp_sums[warp - 1] : 0) + incl - s;
  *total = warp_sums[31];
  __syncthreads();  // warp_sums may be reused at once
  return make_int4(before, before + v.x, before + v.x + v.y, before + v.x + v.y + v.z);
}

__device__ __forceinline__ int4 load4(const int* data, int i, int n) {
  if (i + 3 < n) return *reinterpret_cast<const int4*>(data + i);  // data is 16-byte aligned, i a multiple of 4
  int4 v = make_int4(0, 0, 0, 0);
  if (i < n) v.x = data[i];
  if (i + 1 < n) v.y = data[i + 1];
  if (i + 2 < n) v.z = data[i + 2];
  return v;
}

__device__ __forceinline__ void store4(int* data, int i, int n, int4 v) {
  if (i + 3 < n) {
    *reinterpret_cast<int4*>(data + i) = v;
  } else {
    if (i < n) data[i] = v.x;
    if (i + 1 < n) data[i + 1] = v.y;
    if (i + 2 < n) data[i + 2] = v.z;
  }
}

__global__ void __launch_bounds__(1024) scan_block_sums_kernel(const int* __restrict__ data, int n, int* __restrict__ block_sums) {
  __shared__ int warp_sums[32];
  int total;
  scan_block(load4(data, blockIdx.x * kScanBlock + threadIdx.x * 4, n), warp_sums, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// one CTA, any n: block after block with a running carry (used for the block sums, and for short arrays)
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(int* __restrict__ data, int n, int* __restrict__ total_out) {
  __shared__ int warp_sums[32];
  int carry = 0;
  for (int base = 0; base < n; base += kScanBlock) {
    const int i = base + threadIdx.x * 4;
    int total;
    int4 o = scan_block(load4(data, i, n), warp_sums, &total);
    o.x += carry; o.y += carry; o.z += carry; o.w += carry;
    store4(data, i, n, o);
    carry += total;
  }
  if (threadIdx.x == 0 && total_out) *total_out = carry;
}

__global__ void __launch_bounds__(1024) scan_apply_kernel(int* __restrict__ data, int n, const int* __restrict__ block_offsets) {
  __shared__ int warp_sums[32];
  const int i = blockIdx.x * kScanBlock + threadIdx.x * 4;
  const int off = block_offsets[blockIdx.x];
  int total;
  int4 o = scan_block(load4(data, i, n), warp_sums, &total);
  o.x += off; o.y += off; o.z += off; o.w += off;
  store4(data, i, n, o);
}

static void exclusive_scan(int* data, int n, int* total_out, int* block_sums, cudaStream_t st, int* launches) {
  const int nb = (n + kScanBlock - 1) / kScanBlock;
  if (nb <= 1) {
    exclusive_scan_kernel<<<1, 1024, 0, st>>>(data, n, total_out);
    *launches += 1;
    return;
  }
  scan_block_sums_kernel<<<nb, 1024, 0, st>>>(data, n, block_sums);
  exclusive_scan_kernel<<<1, 1024, 0, st>>>(block_sums, nb, total_out);
  scan_apply_kernel<<<nb, 1024, 0, st>>>(data, n, block_sums);
  *launches += 3;
}

// One warp per tile walks its keys in order, 32 at a time; equal digits inside a round are ranked
// by lane, rounds are sequential, tiles are ordered by the scanned counts: a stable scatter.
template <bool FIRST>
__global__ void __launch_bounds__(32) sort_scatter_kernel(const int64_t* __restrict__ indices, const int* __restrict__ keys_in,
                                                          const int* __restrict__ vals_in, int* __restrict__ keys_out,
                                                          int* __restrict__ vals_out, int n, int F, int shift, int radix,
                                                          int ntiles, const int* __restrict__ offsets) {
  extern __shared__ int base[];
  const int lane = threadIdx.x;
  for (int d = lane; d < radix; d += 32) base[d] = offsets[(size_t)d * ntiles + blockIdx.x];
  __syncwarp();
  const int t0 = blockIdx.x * kSortTile;
  const int t1 = min(n, t0 + kSortTile);
  for (int r = t0; r < t1; r += 32) {
    const int i = r + lane;
    const bool live = i < t1;
    int k = 0, v = 0;
    if (live) {
      if (FIRST) {
        int64_t x = indices[i];
        k = ((uint64_t)x >= (uint64_t)F) ? 0 : (int)x;
        v = i;
      } else {
        k = keys_in[i];
        v = vals_in[i];
      }
    }
    const int d = live ? ((k >> shift) & (radix - 1)) : radix;  // dead lanes match only each other
    const unsigned peers = __match_any_sync(0xffffffffu, d);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int pos = 0;
    if (live) pos = base[d] + rank;
    __syncwarp();
    if (live && rank == 0) base[d] += __popc(peers);
    __syncwarp();
    if (live) {
      keys_out[pos] = k;
      vals_out[pos] = v;
    }
  }
}

// seg_begin[f] = first sorted slot whose key is >= f, for f in [0, F]; slot_of[position] = its slot
__global__ void __launch_bounds__(256) segment_bounds_kernel(const int* __restrict__ keys, const int* __restrict__ order, int n, int F,
                                                             int* __restrict__ seg_begin, int* __restrict__ slot_of) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  const int lo = (i == 0) ? -1 : keys[i - 1];
  const int hi = (i == n) ? F : keys[i];
  for (int f = lo + 1; f <= hi; f++) seg_begin[f] = i;
  if (i < n) slot_of[order[i]] = i;
}

// items per decoder row (>= 1 so that untouched rows still get their zero row written) and, for
// rows cut into several items, how many partial rows they need
__global__ void __launch_bounds__(256) item_counts_kernel(const int* __restrict__ seg_begin, int F, int* __restrict__ item_begin,
                                                          int* __restrict__ part_begin) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  const int cnt = seg_begin[f + 1] - seg_begin[f];
  const int items = max(1, (cnt + kItemSlots - 1) / kItemSlots);
  item_begin[f] = items;
  part_begin[f] = items > 1 ? items : 0;
}

__global__ void __launch_bounds__(256) item_rows_kernel(const int* __restrict__ item_begin, int F, int* __restrict__ item_row) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  for (int i = item_begin[f]; i < item_begin[f + 1]; i++) item_row[i] = f;
}

size_t det_index_bytes(int64_t n, int64_t F) {
  size_t b = 0;
  b += 4 * align256((size_t)n * 4);                                  // keys/vals ping-pong
  b += align256((size_t)2048 * ((n + kSortTile - 1) / kSortTile) * 4);  // digit counts
  b += 3 * align256((size_t)(F + 1) * 4);                            // seg_begin, item_begin, part_begin
  b += align256((size_t)n * 4);                                      // slot_of
  b += align256((size_t)(F + n / kItemSlots + 2) * 4);               // item_row
  b += 256;                                                          // totals
  const size_t longest = (size_t)2048 * ((n + kSortTile - 1) / kSortTile) > (size_t)(F + 1)
                             ? (size_t)2048 * ((n + kSortTile - 1) / kSortTile) : (size_t)(F + 1);
  b += align256(((longest + kScanBlock - 1) / kScanBlock + 4) * 4);  // block sums of the scans
  return b;
}

size_t det_part_rows(int64_t n, int64_t F) { return (size_t)(2 * (n / kItemSlots) + 2); }

cudaError_t det_prepare(const int64_t* indices, int64_t n64, int64_t F64, char* ws, DetIndex* out, cudaStream_t st,
                        int* launches) {
  const int n = (int)n64, F = (int)F64;
  char* p = ws;
  auto take = [&](size_t bytes) { char* q = p; p += align256(bytes); return q; };
  int* keys[2] = {(int*)take((size_t)n * 4), (int*)take((size_t)n * 4)};
  int* vals[2] = {(int*)take((size_t)n * 4), (int*)take((size_t)n * 4)};
  const int ntiles = (n + kSortTile - 1) / kSortTile;
  int* counts = (int*)take((size_t)2048 * ntiles * 4);
  out->seg_begin = (int*)take((size_t)(F + 1) * 4);
  out->item_begin = (int*)take((size_t)(F + 1) * 4);
  out->part_begin = (int*)take((size_t)(F + 1) * 4);
  out->slot_of = (int*)take((size_t)n * 4);
  out->item_row = (int*)take((size_t)(F + n / kItemSlots + 2) * 4);
  int* totals = (int*)take(256);
  const size_t longest = (size_t)2048 * ntiles > (size_t)(F + 1) ? (size_t)2048 * ntiles : (size_t)(F + 1);
  int* block_sums = (int*)take(((longest + kScanBlock - 1) / kScanBlock + 4) * 4);
  out->max_items = F + n / kItemSlots + 1;

  int bits = 1;
  while ((1ll << bits) < F64) bits++;
  const int passes = (bits + 10) / 11;          // digits of at most 11 bits
  const int dbits = (bits + passes - 1) / passes;
  const int radix = 1 << dbits;
  int cur = 0;
  for (int ps = 0; ps < passes; ps++) {
    const int shift = ps * dbits;
    const size_t sh = (size_t)radix * 4;
    if (ps == 0) {
      sort_hist_kernel<true><<<ntiles, 256, sh, st>>>(indices, nullptr, n, F, shift, radix, ntiles, counts);
    } else {
      sort_hist_kernel<false><<<ntiles, 256, sh, st>>>(nullptr, keys[cur], n, F, shift, radix, ntiles, counts);
    }
    exclusive_scan(counts, radix * ntiles, nullptr, block_sums, st, launches);
    if (ps == 0) {
      sort_scatter_kernel<true><<<ntiles, 32, sh, st>>>(indices, nullptr, nullptr, keys[0], vals[0], n, F, shift, radix, ntiles, counts);
      cur = 0;
    } else {
      sort_scatter_kernel<false><<<ntiles, 32, sh, st>>>(nullptr, keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], n, F, shift,
                                                         radix, ntiles, counts);
      cur ^= 1;
    }
    *launches += 2;
  }
  out->order = vals[cur];
  segment_bounds_kernel<<<(n + 1 + 255) / 256, 256, 0, st>>>(keys[cur], vals[cur], n, F, out->seg_begin, out->slot_of);
  item_counts_kernel<<<(F + 255) / 256, 256, 0, st>>>(out->seg_begin, F, out->item_begin, out->part_begin);
  // scans over F + 1 entries (the extra last entry receives the total)
  cudaMemsetAsync(out->item_begin + F, 0, 4, st);
  cudaMemsetAsync(out->part_begin + F, 0, 4, st);
  exclusive_scan(out->item_begin, F + 1, totals, block_sums, st, launches);
  exclusive_scan(out->part_begin, F + 1, totals + 1, block_sums, st, launches);
  item_rows_kernel<<<(F + 255) / 256, 256, 0, st>>>(out->item_begin, F, out->item_row);
  *launches += 3;
  return cudaGetLastError();
}

// ---- ordered segmented sums ----------------------------------------------------------------------
// Level 1: one lane group per item adds its (at most 32) staged rows in slot order.  A decoder row
// with a single item is finished here (converted and written to dweight); otherwise the partial
// row goes to `part` and level 2 adds the row's partials in item order.
template <typename T, int G>
__global__ void __launch_bounds__(128) ordered_sum_items_kernel(const float* __restrict__ stage, const DetIndex ix, int F, int D,
                                                                int piece, float* __restrict__ part, void* __restrict__ dweight) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  const int item = blockIdx.x * (128 / G) + threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int total_items = ix.item_begin[F];
  if (item >= total_items) return;
  const int f = ix.item_row[item];
  const int first = ix.item_begin[f];
  const int items = ix.item_begin[f + 1] - first;
  const int s0 = ix.seg_begin[f] + (item - first) * kItemSlots;
  const int s1 = min(ix.seg_begin[f + 1], s0 + kItemSlots);
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; j++) acc[j] = 0.f;
  const float* src = stage + (size_t)lig * VEC;
  for (int s = s0; s < s1; s += 4) {
    float4 v[4][VEC / 4];
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (s + q < s1) {
#pragma unroll
        for (int h = 0; h < VEC / 4; h++) v[q][h] = __ldcs(reinterpret_cast<const float4*>(src + (size_t)(s + q) * PW) + h);
      }
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (s + q < s1) {
#pragma unroll
        for (int h = 0; h < VEC / 4; h++) {
          acc[4 * h] += v[q][h].x;
          acc[4 * h + 1] += v[q][h].y;
          acc[4 * h + 2] += v[q][h].z;
          acc[4 * h + 3] += v[q][h].w;
        }
      }
  }
  const int col = piece * PW + lig * VEC;
  if (items == 1) {
    if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(dweight) + (size_t)f * D + col) = Pack<T>::pack(acc);
  } else {
    float4* dst = reinterpret_cast<float4*>(part + ((size_t)ix.part_begin[f] + (item - first)) * PW + lig * VEC);
#pragma unroll
    for (int h = 0; h < VEC / 4; h++) dst[h] = make_float4(acc[4 * h], acc[4 * h + 1], acc[4 * h + 2], acc[4 * h + 3]);
  }
}

// Level 2: decoder rows that were cut into several items.
template <typename T, int G>
__global__ void __launch_bounds__(128) ordered_sum_parts_kernel(const float* __restrict__ part, const DetIndex ix, int F, int D,
                                                                int piece, void* __restrict__ dweight) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  const int f = blockIdx.x * (128 / G) + threadIdx.x / G;
  const int lig = threadIdx.x % G;
  if (f >= F) return;
  const int items = ix.item_begin[f + 1] - ix.item_begin[f];
  if (items <= 1) return;
  const float* src = part + (size_t)ix.part_begin[f] * PW + lig * VEC;
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; j++) acc[j] = 0.f;
  for (int s = 0; s < items; s += 4) {
    float4 v[4][VEC / 4];
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (s + q < items) {
#pragma unroll
        for (int h = 0; h < VEC / 4; h++) v[q][h] = *(reinterpret_cast<const float4*>(src + (size_t)(s + q) * PW) + h);
      }
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (s + q < items) {
#pragma unroll
        for (int h = 0; h < VEC / 4; h++) {
          acc[4 * h] += v[q][h].x;
          acc[4 * h + 1] += v[q][h].y;
          acc[4 * h + 2] += v[q][h].z;
          acc[4 * h + 3] += v[q][h].w;
        }
      }
  }
  const int col = piece * PW + lig * VEC;
  if (col < D) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(dweight) + (size_t)f * D + col) = Pack<T>::pack(acc);
}

template <typename T, int G>
static cudaError_t reduce_piece_t(const float* stage, const DetIndex& ix, int F, int D, int piece, float* part, void* dweight,
                                  cudaStream_t st, int* launches) {
  const int per = 128 / G;
  ordered_sum_items_kernel<T, G><<<(ix.max_items + per - 1) / per, 128, 0, st>>>(stage, ix, F, D, piece, part, dweight);
  ordered_sum_parts_kernel<T, G><<<(F + per - 1) / per, 128, 0, st>>>(part, ix, F, D, piece, dweight);
  *launches += 2;
  return cudaGetLastError();
}

cudaError_t det_reduce_piece(int wdt, int G, const float* stage, const DetIndex& ix, int F, int D, int piece, float* part,
                             void* dweight, cudaStream_t st, int* launches) {
#define CALL_G(T)                                                                                     \
  (G == 32 ? reduce_piece_t<T, 32>(stage, ix, F, D, piece, part, dweight, st, launches)                \
           : (G == 16 ? reduce_piece_t<T, 16>(stage, ix, F, D, piece, part, dweight, st, launches)     \
                      : reduce_piece_t<T, 8>(stage, ix, F, D, piece, part, dweight, st, launches)))
  if (wdt == FLEXSAE_F32) return CALL_G(float);
  if (wdt == FLEXSAE_BF16) return CALL_G(__nv_bfloat16);
  return CALL_G(__half);
#undef CALL_G
}

}  // namespace flexsae
