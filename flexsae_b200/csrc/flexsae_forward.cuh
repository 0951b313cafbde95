// Forward kernels of the fused decoder losses: gather, running K-prefix residual, squared error.
#pragma once

#include "flexsae_kernel_args.cuh"

namespace flexsae {

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

}  // namespace flexsae
