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
#include <stdio.h>
#include <string.h>

#include "flexsae_common.cuh"

namespace flexsae {

// ---- tuning state ------------------------------------------------------------------------------
struct Options {
  int lanes_fwd = 0;      // 0 = auto
  int lanes_bwd = 0;      // 0 = auto
  int l2_budget_mb = 96;  // bytes of one piece's decoder columns (+ fp32 slab) kept under this
  int slab_pieces = 1;    // column pieces accumulated per backward launch
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

// warps per CTA for a lane-group width: 8 batch rows (G=32) or 16 (G=16, G=8) per CTA
__host__ __device__ constexpr int warps_per_cta(int G) { return G == 8 ? 4 : 8; }
__host__ __device__ constexpr int rows_per_cta(int G) { return warps_per_cta(G) * (32 / G); }

constexpr int kUnroll = 8;  // decoder-row loads in flight per lane

struct FwdArgs {
  const int64_t* indices;
  const void* weight;
  const void* vals;
  const void* bias;
  const void* target;
  float* loss_part;  // [pieces, B]
  float* resid;      // [B, D]
  int32_t* status;
  int B, K, F, D;
  int vals_dtype, bias_dtype, target_dtype;
};

struct BwdArgs {
  const int64_t* indices;
  const void* weight;
  const void* vals;
  const float* resid;     // [B, D]
  const float* grad_out;  // device scalar
  float* slab;            // [slab_pieces, F, PW] fp32, zero on entry
  float* dv_part;         // [pieces, B, K]
  float* db_part;         // [row tiles, D]
  int32_t* status;
  int B, K, F, D;
  int vals_dtype;
  int piece0;   // first column piece of this launch
  float scale;  // 2 * inv_norm
};

// Stage the CTA's indices (as int32, range-checked) and vals (as fp32) in shared memory.
template <int RPC>
__device__ __forceinline__ void stage_rows(const int64_t* __restrict__ indices, const void* __restrict__ vals,
                                           int vals_dtype, int row0, int B, int K, int F, int* sidx,
                                           float* sval, int32_t* status) {
  const int n = RPC * K;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int r = i / K;
    const int b = row0 + r;
    int id = 0;
    float v = 0.f;
    if (b < B) {
      const size_t g = (size_t)row0 * K + i;
      int64_t x = indices[g];
      if ((uint64_t)x >= (uint64_t)F) {  // never dereference an index outside the table
        x = 0;
        if (status) atomicOr(status, FLEXSAE_STATUS_BAD_INDEX);
      }
      id = (int)x;
      v = load_scalar(vals, vals_dtype, g);
    }
    sidx[i] = id;
    sval[i] = v;
  }
}

// ---- forward -----------------------------------------------------------------------------------
template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(warps_per_cta(G) * 32)
    decoder_loss_fwd_kernel(const FwdArgs a) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int RPC = rows_per_cta(G);
  constexpr int U = kUnroll;
  extern __shared__ int smem_i[];
  int* sidx = smem_i;
  float* sval = reinterpret_cast<float*>(smem_i + RPC * a.K);

  const int row0 = blockIdx.x * RPC;
  const int piece = blockIdx.y;
  stage_rows<RPC>(a.indices, a.vals, a.vals_dtype, row0, a.B, a.K, a.F, sidx, sval, a.status);
  __syncthreads();

  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int b = row0 + gid;
  const int col = piece * PW + lig * VEC;
  const bool active = (b < a.B) && (col < a.D);

  float r[VEC], acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; j++) {
    r[j] = 0.f;
    acc[j] = 0.f;
  }
  if (active) {
    float bv[VEC], tv[VEC];
    load_elems<VEC>(a.bias, a.bias_dtype, (size_t)col, bv);
    load_elems<VEC>(a.target, a.target_dtype, (size_t)b * a.D + col, tv);
#pragma unroll
    for (int j = 0; j < VEC; j++) r[j] = bv[j] - tv[j];
  }

  const char* wcol = reinterpret_cast<const char*>(a.weight) + (size_t)col * sizeof(T);
  const size_t row_bytes = (size_t)a.D * sizeof(T);
  const int* myidx = sidx + gid * a.K;
  const float* myval = sval + gid * a.K;
  const int K = a.K;

  for (int k0 = 0; k0 < K; k0 += U) {
    uint4 w[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      w[u] = make_uint4(0u, 0u, 0u, 0u);
      if (active && k0 + u < K) w[u] = ld_row_piece(wcol + (size_t)myidx[k0 + u] * row_bytes);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (k0 + u < K) {
        const float v = myval[k0 + u];
        float wf[VEC];
        Pack<T>::unpack(w[u], wf);
#pragma unroll
        for (int j = 0; j < VEC; j++) {
          r[j] = fmaf(v, wf[j], r[j]);                    // residual of the k-th prefix
          if (HIER) acc[j] = fmaf(r[j], r[j], acc[j]);   // every prefix is penalised
        }
      }
    }
  }
  if (!HIER) {
#pragma unroll
    for (int j = 0; j < VEC; j++) acc[j] = r[j] * r[j];
  }
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VEC; j++) s += acc[j];
  s = group_sum<G>(s);
  if (lig == 0 && b < a.B) a.loss_part[(size_t)piece * a.B + b] = s;
  if (active) {
    float4* out = reinterpret_cast<float4*>(a.resid + (size_t)b * a.D + col);
#pragma unroll
    for (int i = 0; i < VEC / 4; i++) out[i] = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
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
// Slab column order: a lane's elements 0..3 live at column lig*4 and, for 8-element packs,
// elements 4..7 at column G*4 + lig*4, so that each red.v4 instruction of a lane group covers
// whole contiguous 32-byte sectors (a lane-contiguous 32-byte layout would make every sector
// the target of two separate instructions and halve the L2 atomic throughput).
template <typename T, int G, bool HIER>
__global__ void __launch_bounds__(warps_per_cta(G) * 32)
    decoder_loss_bwd_kernel(const BwdArgs a) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  constexpr int RPC = rows_per_cta(G);
  constexpr int U = kUnroll;
  extern __shared__ int smem_i[];
  int* sidx = smem_i;
  float* sval = reinterpret_cast<float*>(smem_i + RPC * a.K);

  const int row0 = blockIdx.x * RPC;
  const int piece = a.piece0 + blockIdx.y;
  stage_rows<RPC>(a.indices, a.vals, a.vals_dtype, row0, a.B, a.K, a.F, sidx, sval, a.status);
  __syncthreads();

  const int gid = threadIdx.x / G;
  const int lig = threadIdx.x % G;
  const int b = row0 + gid;
  const int col = piece * PW + lig * VEC;
  const bool active = (b < a.B) && (col < a.D);
  const float coef = __ldg(a.grad_out) * a.scale;

  float r[VEC], suf[VEC];
#pragma unroll
  for (int j = 0; j < VEC; j++) r[j] = 0.f;
  if (active) {
    const float4* in = reinterpret_cast<const float4*>(a.resid + (size_t)b * a.D + col);
#pragma unroll
    for (int i = 0; i < VEC / 4; i++) {
      float4 t = __ldg(in + i);
      r[4 * i] = t.x;
      r[4 * i + 1] = t.y;
      r[4 * i + 2] = t.z;
      r[4 * i + 3] = t.w;
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; j++) suf[j] = HIER ? 0.f : r[j];

  const char* wcol = reinterpret_cast<const char*>(a.weight) + (size_t)col * sizeof(T);
  const size_t row_bytes = (size_t)a.D * sizeof(T);
  const int* myidx = sidx + gid * a.K;
  const float* myval = sval + gid * a.K;
  const int K = a.K;
  float* slab = a.slab + (size_t)blockIdx.y * a.F * PW + lig * 4;
  float* dv = a.dv_part + ((size_t)piece * a.B + (b < a.B ? b : 0)) * K;

  for (int kb = K - 1; kb >= 0; kb -= U) {
    uint4 w[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      w[u] = make_uint4(0u, 0u, 0u, 0u);
      if (active && kb - u >= 0) w[u] = ld_row_piece(wcol + (size_t)myidx[kb - u] * row_bytes);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int k = kb - u;
      if (k >= 0) {
        const float v = myval[k];
        const float c = v * coef;
        float wf[VEC];
        Pack<T>::unpack(w[u], wf);
        if (HIER) {
#pragma unroll
          for (int j = 0; j < VEC; j++) suf[j] += r[j];  // S_k = sum_{j>=k} residual_j
        }
        if (active) {
          float* dst = slab + (size_t)myidx[k] * PW;
          red_add_v4(dst, suf[0] * c, suf[1] * c, suf[2] * c, suf[3] * c);
          if (VEC == 8) red_add_v4(dst + G * 4, suf[VEC - 4] * c, suf[VEC - 3] * c, suf[VEC - 2] * c, suf[VEC - 1] * c);
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < VEC; j++) dot = fmaf(wf[j], suf[j], dot);
        dot = group_sum<G>(dot);
        if (lig == 0 && b < a.B) dv[k] = dot * coef;
        if (HIER) {
#pragma unroll
          for (int j = 0; j < VEC; j++) r[j] = fmaf(-v, wf[j], r[j]);  // step back to prefix k-1
        }
      }
    }
  }

  // dbias: column sums of S_0 over this CTA's rows, one partial row per row tile
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_i);  // [RPC][PW], aliases the staged indices
#pragma unroll
  for (int j = 0; j < VEC; j++) red[gid * PW + lig * VEC + j] = suf[j];
  __syncthreads();
  if ((int)threadIdx.x < PW) {
    const int c = piece * PW + threadIdx.x;
    if (c < a.D) {
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < RPC; g++) s += red[g * PW + threadIdx.x];
      a.db_part[(size_t)blockIdx.x * a.D + c] = s * coef;
    }
  }
}

// fp32 slab -> dweight columns of one piece in the decoder's storage type; clears the slab.
template <typename T, int G>
__global__ void __launch_bounds__(256) slab_to_dweight_kernel(float* __restrict__ slab, void* __restrict__ dweight, int F, int D,
                                                              int piece0, int npieces) {
  constexpr int VEC = Pack<T>::VEC;
  constexpr int PW = G * VEC;
  const size_t total = (size_t)npieces * F * G;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int lig = (int)(i % G);
    const size_t fr = i / G;  // piece-in-launch * F + f
    const int pl = (int)(fr / F);
    const int f = (int)(fr - (size_t)pl * F);
    float* s = slab + fr * PW + lig * 4;
    float v[VEC];
    float4 t0 = *reinterpret_cast<float4*>(s);
    v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w;
    *reinterpret_cast<float4*>(s) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC == 8) {
      float4 t1 = *reinterpret_cast<float4*>(s + G * 4);
      v[VEC - 4] = t1.x; v[VEC - 3] = t1.y; v[VEC - 2] = t1.z; v[VEC - 1] = t1.w;
      *reinterpret_cast<float4*>(s + G * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int col = (piece0 + pl) * PW + lig * VEC;
    if (col < D) {
      uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<T*>(dweight) + (size_t)f * D + col);
      *out = Pack<T>::pack(v);
    }
  }
}

// dvals = sum over column pieces (fixed order), dbias = sum over row tiles (fixed order).
__global__ void __launch_bounds__(256) grads_finalize_kernel(const float* __restrict__ dv_part, int pieces, size_t BK,
                                                            void* __restrict__ dvals, int vals_dtype,
                                                            const float* __restrict__ db_part, int tiles, int D,
                                                            void* __restrict__ dbias, int bias_dtype, int dv_blocks) {
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
      for (int t = 0; t < tiles; t++) s += db_part[(size_t)t * D + d];
      store_scalar(dbias, bias_dtype, (size_t)d, s);
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
  if (s.F > (1ll << 30) || s.D > (1ll << 20) || s.B > (1ll << 30) || s.B * s.K > (1ll << 31) - 1)
    return fail(FLEXSAE_EUNSUPPORTED, "shape too large for 32-bit row/position arithmetic");
  // indices and vals of a CTA's rows are staged in shared memory: 16 rows * K * 8 bytes
  if (s.K > 1600) return fail(FLEXSAE_EUNSUPPORTED, "K=%lld above the supported maximum of 1600", (long long)s.K);
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

struct BwdPlan {
  int G, PW, pieces, tiles, slab_pieces;
  size_t off_slab, off_dv, off_db, total;
};

static BwdPlan plan_bwd(const Shape& s, int wdt) {
  BwdPlan p;
  const int vec = 16 / (int)dtype_size(wdt);
  p.G = choose_lanes(s.F, wdt, true, g_opt.lanes_bwd);
  p.PW = p.G * vec;
  p.pieces = (int)((s.D + p.PW - 1) / p.PW);
  p.tiles = (int)((s.B + rows_per_cta(p.G) - 1) / rows_per_cta(p.G));
  p.slab_pieces = g_opt.slab_pieces < 1 ? 1 : (g_opt.slab_pieces > p.pieces ? p.pieces : g_opt.slab_pieces);
  size_t off = 0;
  p.off_slab = off;
  off = align_up(off + (size_t)p.slab_pieces * s.F * p.PW * 4, 256);
  p.off_dv = off;
  off = align_up(off + (size_t)p.pieces * s.B * s.K * 4, 256);
  p.off_db = off;
  off = align_up(off + (size_t)p.tiles * s.D * 4, 256);
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

template <typename T, int G, bool HIER>
static cudaError_t launch_fwd(const FwdArgs& a, int pieces, cudaStream_t st) {
  constexpr int RPC = rows_per_cta(G);
  const size_t smem = (size_t)RPC * a.K * 8;
  auto kern = decoder_loss_fwd_kernel<T, G, HIER>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  dim3 grid((a.B + RPC - 1) / RPC, pieces);
  kern<<<grid, warps_per_cta(G) * 32, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G, bool HIER>
static cudaError_t launch_bwd(const BwdArgs& a, int npieces, cudaStream_t st) {
  constexpr int RPC = rows_per_cta(G);
  constexpr int PW = G * Pack<T>::VEC;
  size_t smem = (size_t)RPC * a.K * 8;
  if (smem < (size_t)RPC * PW * 4) smem = (size_t)RPC * PW * 4;
  auto kern = decoder_loss_bwd_kernel<T, G, HIER>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  dim3 grid((a.B + RPC - 1) / RPC, npieces);
  kern<<<grid, warps_per_cta(G) * 32, smem, st>>>(a);
  t_launches++;
  return cudaGetLastError();
}

template <typename T, int G>
static cudaError_t launch_convert(float* slab, void* dweight, int F, int D, int piece0, int npieces, cudaStream_t st) {
  const size_t total = (size_t)npieces * F * G;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  slab_to_dweight_kernel<T, G><<<(unsigned)blocks, 256, 0, st>>>(slab, dweight, F, D, piece0, npieces);
  t_launches++;
  return cudaGetLastError();
}

// dispatch over (element type, lanes, loss kind)
#define FLEXSAE_DISPATCH_G(T, G, kind, CALL)          \
  ((kind) == FLEXSAE_HIER ? CALL(T, G, true) : CALL(T, G, false))
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

int flexsae_version(void) { return 100; }

const char* flexsae_last_error(void) { return t_err; }

int flexsae_last_launch_count(void) { return t_launches; }

int flexsae_set_option(const char* name, int64_t value) {
  if (!name) return fail(FLEXSAE_EINVAL, "option name is null");
  const bool lanes_ok = value == 0 || value == 8 || value == 16 || value == 32;
  if (!strcmp(name, "lanes_fwd") && lanes_ok) { g_opt.lanes_fwd = (int)value; return 0; }
  if (!strcmp(name, "lanes_bwd") && lanes_ok) { g_opt.lanes_bwd = (int)value; return 0; }
  if (!strcmp(name, "l2_budget_mb") && value >= 1 && value <= 4096) { g_opt.l2_budget_mb = (int)value; return 0; }
  if (!strcmp(name, "slab_pieces") && value >= 1 && value <= 65535) { g_opt.slab_pieces = (int)value; return 0; }
  return fail(FLEXSAE_EINVAL, "unknown option or value: %s=%lld", name, (long long)value);
}

int64_t flexsae_get_option(const char* name) {
  if (!name) return -1;
  if (!strcmp(name, "lanes_fwd")) return g_opt.lanes_fwd;
  if (!strcmp(name, "lanes_bwd")) return g_opt.lanes_bwd;
  if (!strcmp(name, "l2_budget_mb")) return g_opt.l2_budget_mb;
  if (!strcmp(name, "slab_pieces")) return g_opt.slab_pieces;
  return -1;
}

size_t flexsae_fwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  return plan_fwd(s, weight_dtype).total;
}

size_t flexsae_bwd_workspace_bytes(int kind, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype, int dw_mode) {
  Shape s{B, K, F, D};
  if (check_shape(kind, s, weight_dtype)) return 0;
  if (dw_mode != FLEXSAE_DW_ATOMIC) return 0;
  return plan_bwd(s, weight_dtype).total;
}

int flexsae_loss_fwd(int kind, const int64_t* indices, const void* weight, const void* vals, const void* bias,
                     const void* target, float* loss_out, float* resid_out, void* workspace, size_t workspace_bytes,
                     int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype, int vals_dtype, int bias_dtype,
                     int target_dtype, double inv_norm, int32_t* status, void* stream) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype) || !dtype_ok(target_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d, target %d)", vals_dtype, bias_dtype, target_dtype);
  if (!indices || !weight || !vals || !bias || !target || !loss_out || !resid_out || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(bias) || !aligned16(target) || !aligned16(resid_out) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, bias, target, resid and workspace must be 16-byte aligned");
  const FwdPlan p = plan_fwd(s, weight_dtype);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "forward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  FwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.bias = bias; a.target = target;
  a.loss_part = reinterpret_cast<float*>(workspace);
  a.resid = resid_out; a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype; a.bias_dtype = bias_dtype; a.target_dtype = target_dtype;

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

int flexsae_loss_bwd(int kind, const int64_t* indices, const void* weight, const void* vals, const float* resid,
                     const float* grad_out, void* dweight, void* dvals, void* dbias, void* workspace,
                     size_t workspace_bytes, int64_t B, int64_t K, int64_t F, int64_t D, int weight_dtype,
                     int vals_dtype, int bias_dtype, double inv_norm, int dw_mode, int32_t* status, void* stream) {
  t_launches = 0;
  Shape s{B, K, F, D};
  if (int rc = check_shape(kind, s, weight_dtype)) return rc;
  if (!dtype_ok(vals_dtype) || !dtype_ok(bias_dtype))
    return fail(FLEXSAE_EINVAL, "unknown dtype code (vals %d, bias %d)", vals_dtype, bias_dtype);
  if (dw_mode != FLEXSAE_DW_ATOMIC)
    return fail(FLEXSAE_EUNSUPPORTED, "dweight mode %d is not available", dw_mode);
  if (!indices || !weight || !vals || !resid || !grad_out || !dweight || !dvals || !dbias || !workspace)
    return fail(FLEXSAE_EINVAL, "null pointer argument");
  if (!aligned16(weight) || !aligned16(resid) || !aligned16(dweight) || !aligned16(workspace))
    return fail(FLEXSAE_EINVAL, "weight, resid, dweight and workspace must be 16-byte aligned");
  const BwdPlan p = plan_bwd(s, weight_dtype);
  if (workspace_bytes < p.total)
    return fail(FLEXSAE_EWORKSPACE, "backward workspace too small: %zu < %zu bytes", workspace_bytes, p.total);
  if (inv_norm <= 0.0) inv_norm = 1.0 / ((double)B * (double)D * (kind == FLEXSAE_HIER ? (double)K : 1.0));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char* ws = reinterpret_cast<char*>(workspace);

  BwdArgs a;
  a.indices = indices; a.weight = weight; a.vals = vals; a.resid = resid; a.grad_out = grad_out;
  a.slab = reinterpret_cast<float*>(ws + p.off_slab);
  a.dv_part = reinterpret_cast<float*>(ws + p.off_dv);
  a.db_part = reinterpret_cast<float*>(ws + p.off_db);
  a.status = status;
  a.B = (int)B; a.K = (int)K; a.F = (int)F; a.D = (int)D;
  a.vals_dtype = vals_dtype;
  a.scale = (float)(2.0 * inv_norm);

  // The slab is cleared once here; afterwards every conversion pass leaves it cleared.
  cudaError_t e = cudaMemsetAsync(a.slab, 0, (size_t)p.slab_pieces * F * p.PW * 4, st);
  if (e != cudaSuccess) return fail((int)e, "slab clear failed: %s", cudaGetErrorString(e));
  for (int p0 = 0; p0 < p.pieces; p0 += p.slab_pieces) {
    const int np = (p.pieces - p0 < p.slab_pieces) ? p.pieces - p0 : p.slab_pieces;
    a.piece0 = p0;
#define CALL_BWD(T, G, H) launch_bwd<T, G, H>(a, np, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_BWD);
#undef CALL_BWD
    if (e != cudaSuccess) return fail((int)e, "backward launch failed: %s", cudaGetErrorString(e));
#define CALL_CVT(T, G, H) launch_convert<T, G>(a.slab, dweight, (int)F, (int)D, p0, np, st)
    e = FLEXSAE_DISPATCH(weight_dtype, p.G, kind, CALL_CVT);
#undef CALL_CVT
    if (e != cudaSuccess) return fail((int)e, "slab conversion launch failed: %s", cudaGetErrorString(e));
  }
  const size_t BK = (size_t)B * K;
  const int dv_blocks = (int)((BK + 255) / 256);
  const int db_blocks = (int)((D + 255) / 256);
  grads_finalize_kernel<<<dv_blocks + db_blocks, 256, 0, st>>>(a.dv_part, p.pieces, BK, dvals, vals_dtype, a.db_part,
                                                             p.tiles, (int)D, dbias, bias_dtype, dv_blocks);
  t_launches++;
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "gradient finalize launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
