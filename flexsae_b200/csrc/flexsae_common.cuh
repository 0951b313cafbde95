// Shared device helpers of the decoder-loss kernels: 16-byte row-piece loads, element-type
// conversion, vectorised reductions into global memory, small group reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flexsae_b200.h"

namespace flexsae {

// ---- element packs: one 16-byte load per lane ------------------------------------------------
template <typename T>
struct Pack;

template <>
struct Pack<float> {
  static constexpr int VEC = 4;
  static constexpr int DTYPE = FLEXSAE_F32;
  __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ __forceinline__ static void unpack_pairs(const uint4& u, float2* f) {
    f[0] = make_float2(__uint_as_float(u.x), __uint_as_float(u.y));
    f[1] = make_float2(__uint_as_float(u.z), __uint_as_float(u.w));
  }
};

template <>
struct Pack<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static constexpr int DTYPE = FLEXSAE_BF16;
  // bf16 -> fp32 is a 16-bit shift: two integer ops per pair, no conversion unit involved
  __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x << 16);
    f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16);
    f[3] = __uint_as_float(u.y & 0xffff0000u);
    f[4] = __uint_as_float(u.z << 16);
    f[5] = __uint_as_float(u.z & 0xffff0000u);
    f[6] = __uint_as_float(u.w << 16);
    f[7] = __uint_as_float(u.w & 0xffff0000u);
  }
  __device__ __forceinline__ static void unpack_pairs(const uint4& u, float2* f) {
    f[0] = make_float2(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u));
    f[1] = make_float2(__uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
    f[2] = make_float2(__uint_as_float(u.z << 16), __uint_as_float(u.z & 0xffff0000u));
    f[3] = make_float2(__uint_as_float(u.w << 16), __uint_as_float(u.w & 0xffff0000u));
  }
  __device__ __forceinline__ static uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};

template <>
struct Pack<__half> {
  static constexpr int VEC = 8;
  static constexpr int DTYPE = FLEXSAE_F16;
  __device__ __forceinline__ static void unpack2(uint32_t w, float* f) {
    float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w));
    f[0] = t.x;
    f[1] = t.y;
  }
  __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
    unpack2(u.x, f);
    unpack2(u.y, f + 2);
    unpack2(u.z, f + 4);
    unpack2(u.w, f + 6);
  }
  __device__ __forceinline__ static void unpack_pairs(const uint4& u, float2* f) {
    f[0] = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    f[1] = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    f[2] = __half22float2(*reinterpret_cast<const __half2*>(&u.z));
    f[3] = __half22float2(*reinterpret_cast<const __half2*>(&u.w));
  }
  __device__ __forceinline__ static uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};

// ---- memory instructions -----------------------------------------------------------------------
// One 16-byte piece of a gathered decoder row.  A plain (L1-allocating) load on purpose: measured
// on B200, `ld.global.nc.L1::no_allocate` tops out near 9.5 TB/s from L2 and its lines are not
// retained in L2 between the ~8 batch rows that use the same decoder row (4.5x the table in HBM
// reads per pass), while the plain load reaches ~15 TB/s and keeps the column piece L2-resident.
__device__ __forceinline__ uint4 ld_row_piece(const void* p) {
  uint4 v;
  asm("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Asynchronous 16-byte global -> shared copy (L2 only); `bytes` = 16 copies, 0 writes zeros
// without touching global memory.  Completion is tracked per thread in commit groups.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// 16-byte fire-and-forget fp32 add, resolved by the L2 atomic units (sm_90+).
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// ---- NVLink SHARP (multimem) on a multicast address: the switch sums the same 16 bytes of every
// GPU's replica (fp32 accumulation for 16-bit types) / stores 16 bytes into every replica.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce(const void* mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<float>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<__nv_bfloat16>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<__half>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// ---- run-time typed loads / stores for the small operands (vals, bias, target) -------------
__device__ __forceinline__ float load_scalar(const void* p, int dtype, size_t i) {
  if (dtype == FLEXSAE_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == FLEXSAE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_scalar(void* p, int dtype, size_t i, float v) {
  if (dtype == FLEXSAE_F32)
    reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == FLEXSAE_BF16)
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// N (4 or 8) consecutive elements starting at element offset `off` (a multiple of N), widened.
template <int N>
__device__ __forceinline__ void load_elems(const void* p, int dtype, size_t off, float* out) {
  if (dtype == FLEXSAE_F32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + off);
#pragma unroll
    for (int i = 0; i < N / 4; i++) {
      float4 t = __ldg(q + i);
      out[4 * i] = t.x;
      out[4 * i + 1] = t.y;
      out[4 * i + 2] = t.z;
      out[4 * i + 3] = t.w;
    }
  } else {
    const uint2* q = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p) + off);
#pragma unroll
    for (int i = 0; i < N / 4; i++) {
      uint2 t = __ldg(q + i);
      if (dtype == FLEXSAE_BF16) {
        out[4 * i] = __uint_as_float(t.x << 16);
        out[4 * i + 1] = __uint_as_float(t.x & 0xffff0000u);
        out[4 * i + 2] = __uint_as_float(t.y << 16);
        out[4 * i + 3] = __uint_as_float(t.y & 0xffff0000u);
      } else {
        Pack<__half>::unpack2(t.x, out + 4 * i);
        Pack<__half>::unpack2(t.y, out + 4 * i + 2);
      }
    }
  }
}

// Packed fp32 arithmetic (two lanes of a 64-bit register pair per instruction, sm_100): the
// kernels are bound by instruction issue as much as by memory, and this halves the FP32 issue slots.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }

// Sum over the G lanes (G = 8, 16 or 32, lane groups aligned to G) that share one batch row.
template <int G>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int m = G / 2; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

}  // namespace flexsae
