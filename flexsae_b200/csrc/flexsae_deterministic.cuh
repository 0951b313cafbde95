// Internal interface between the loss kernels and the deterministic-dweight support code.
#pragma once

#include "flexsae_common.cuh"

namespace flexsae {

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Sorted view of the B*K (decoder row, position) pairs; all pointers are device memory carved
// out of the caller's workspace.
struct DetIndex {
  int* order;       // [n]   position (b*K+k) held by each sorted slot
  int* slot_of;     // [n]   sorted slot of each position (inverse of order)
  int* seg_begin;   // [F+1] first slot of each decoder row
  int* item_begin;  // [F+1] first item of each decoder row (items = runs of at most 32 slots)
  int* part_begin;  // [F+1] first partial row of each decoder row that has more than one item
  int* item_row;    // [items] decoder row of each item
  int max_items;    // upper bound on the number of items (grid size)
};

size_t det_index_bytes(int64_t n, int64_t F);  // workspace of det_prepare
size_t det_part_rows(int64_t n, int64_t F);    // rows of the partial-sum buffer (each PW floats)

// Sorts the pairs and builds the index (about a dozen small launches on `st`).
cudaError_t det_prepare(const int64_t* indices, int64_t n, int64_t F, char* ws, DetIndex* out, cudaStream_t st,
                        int* launches);

// dweight[:, piece columns] = ordered sums of the staged rows [n, PW] of one column piece.
cudaError_t det_reduce_piece(int wdt, int G, const float* stage, const DetIndex& ix, int F, int D, int piece, float* part,
                             void* dweight, cudaStream_t st, int* launches);

}  // namespace flexsae
