// Shared host/device helpers for the torchair-b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/tab_api.h"

namespace tab {

// Records a formatted message for tab_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

inline cudaStream_t as_stream(tab_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Reports a failed launch (bad configuration and the like) without synchronising; on success adds `kernels` to the
// process-wide count of kernels this library has enqueued (tab_launch_count).
int check_launch(const char* what, int kernels = 1);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Grid size for a grid-stride kernel: enough CTAs to fill the machine `waves` times, never more than the work.
inline int grid_for(int64_t work_items, int ctas_per_sm) {
  int64_t cap = static_cast<int64_t>(kNumSMs) * ctas_per_sm;
  int64_t g = work_items < cap ? work_items : cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

// ---- element loads: 8 consecutive elements (16 bytes of 16-bit data, 32 bytes of fp32) as fp32 ----
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};

template <>
struct Elem<__half> {
  static __device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store8(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};

template <>
struct Elem<float> {
  static __device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  static __device__ __forceinline__ float to_f32(float x) { return x; }
  static __device__ __forceinline__ float from_f32(float x) { return x; }
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Symmetric int8 quantisation of one value given its row scale: IEEE division, round-half-even,
// clamp to +-127.  scale == 0 (all-zero row) gives 0.
__device__ __forceinline__ int quant_i8(float v, float scale) {
  if (!(scale > 0.f)) return 0;
  int q = __float2int_rn(__fdiv_rn(v, scale));
  return max(-127, min(127, q));
}

__device__ __forceinline__ uint32_t pack4_i8(int a, int b, int c, int d) {
  return (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8) |
         ((static_cast<uint32_t>(c) & 0xffu) << 16) | ((static_cast<uint32_t>(d) & 0xffu) << 24);
}

// IEEE reciprocal RN(1/d) of a normal d whose reciprocal is normal too (here d = 1 + e lies in [1, 5.6e34]): the
// hardware seed followed by one Newton step in FMAs.  On sm_100 this equals the correctly rounded reciprocal for every
// one of the 2^23 significands (checked exhaustively against the library's IEEE reciprocal by tab_selftest_reciprocal,
// which the GPU tests run); scaling by a power of two changes no step, so it holds for every exponent in range.  Two
// FMAs instead of the library's checked sequence with its out-of-line slow path.
__device__ __forceinline__ float rcp_rn_normal(float d) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d));   // d and 1/d are normal: the flush-to-zero form is the bare seed instruction
  return __fmaf_rn(__fmaf_rn(-d, y, 1.0f), y, y);
}

// silu(a) * b = RN(RN(a * RN(1 / (1 + e))) * b) in fp32 with e = exp(-a) from a fixed sequence of correctly rounded
// operations (two FMAs of range reduction with the rounded log2(e), a degree-6 polynomial for 2^f on [-0.5, 0.5] in
// Horner form, the integer part added into the exponent field, the IEEE reciprocal), so that a CPU restatement of the
// same sequence gives the same bits: int8 values quantised after SwiGLU then do not depend on whose exp() was used.  e
// is within 1.3 ulp of exp(-a) apart from the rounded log2(e) (relative error |a| * 1.3e-8).  -a is capped to
// [-80, 80]: beyond it 1 + e is 1, or the result is below 1e-33 in magnitude.  20 instructions, no branch.
// Building with -DTAB_FAST_SILU swaps in the earlier form (hardware ex2.approx and an approximate reciprocal with one
// remainder correction: half the instructions, results within a few ulp but not reproducible on a CPU).
constexpr float kLog2e = 0x1.715476p+0f;
constexpr float kRoundMagicF = 12582912.0f;   // 1.5 * 2^23
__device__ __forceinline__ float silu_mul(float a, float b) {
#ifdef TAB_FAST_SILU
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(fminf(-a, 80.0f), 1.4426950408889634f)));
  const float d = __fadd_rn(1.0f, e);
  float y;
  asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(d));
  const float q0 = __fmul_rn(a, y);
  const float r = __fmaf_rn(-q0, d, a);
  const float s = __fmaf_rn(r, y, q0);
  return __fmul_rn(s, b);
#else
  const float x = fminf(fmaxf(-a, -80.0f), 80.0f);
  const float nm = __fmaf_rn(x, kLog2e, kRoundMagicF);     // integer n = rint(x * log2e) in the low mantissa bits
  const float n = __fadd_rn(nm, -kRoundMagicF);
  const float f = __fmaf_rn(x, kLog2e, -n);                 // |f| <= 0.5
  float p = 0x1.41d334p-13f;
  p = __fmaf_rn(p, f, 0x1.5f456ap-10f);
  p = __fmaf_rn(p, f, 0x1.3b2dbcp-7f);
  p = __fmaf_rn(p, f, 0x1.c6aed4p-5f);
  p = __fmaf_rn(p, f, 0x1.ebfbdap-3f);
  p = __fmaf_rn(p, f, 0x1.62e430p-1f);
  p = __fmaf_rn(p, f, 1.0f);
  const float e = __uint_as_float(__float_as_uint(p) + (__float_as_uint(nm) << 23));   // p * 2^n
  const float d = __fadd_rn(1.0f, e);
  return __fmul_rn(__fmul_rn(a, rcp_rn_normal(d)), b);
#endif
}


// ---- raw (unconverted) storage of 8 consecutive elements, to keep a row in few registers between passes ----
template <typename T>
struct Raw8 {
  uint4 r;
  __device__ __forceinline__ void load(const T* p) { r = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void unpack(float (&v)[8]) const;
};

template <>
__device__ __forceinline__ void Raw8<__nv_bfloat16>::unpack(float (&v)[8]) const {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <>
__device__ __forceinline__ void Raw8<__half>::unpack(float (&v)[8]) const {
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <>
struct Raw8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void unpack(float (&v)[8]) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

// Maximum over the CTA; `red` holds one float per warp.  All threads must call it.
template <int THREADS>
__device__ __forceinline__ float cta_max(float v, float* red) {
  v = warp_max(v);
  if constexpr (THREADS == 32) return v;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < THREADS / 32 ? red[lane] : 0.f;
  r = warp_max(r);
  __syncthreads();
  return r;
}

// ---- fast exact row quantiser ------------------------------------------------------------------------------
// Produces rint(v / scale) clamped to +-127 -- bit for bit what IEEE division gives -- in four full-rate FP32
// instructions per element, without branches (conversion instructions issue at 1/8 rate, and the library division is a
// dozen instructions with a slow path):
//   * one correctly rounded reciprocal per row, inv = RN(1/scale);
//   * q0 = RN(v * inv); r = fma(-q0, scale, v) is the exact remainder; q1 = fma(r, inv, q0) is then the correctly
//     rounded quotient RN(v / scale) (Markstein's correction step; it needs a correctly rounded reciprocal and fails
//     only for a divisor whose significand is all ones, which is sent down the library path together with scales too
//     small for a finite reciprocal or an exact remainder);
//   * adding 1.5 * 2^23 rounds q1 half-to-even and leaves the integer in the low mantissa bits (its low byte is the
//     two's-complement int8).  |v| <= amax keeps |q1| <= 127, so no clamp is needed.
struct RowQuant {
  float scale, inv;
  bool exact;   // every element takes the library's IEEE division
};

__device__ __forceinline__ RowQuant make_row_quant(float amax) {
  RowQuant rq;
  rq.scale = __fdiv_rn(amax, 127.0f);
  rq.inv = __frcp_rn(rq.scale);
  rq.exact = !(rq.scale > 1e-28f) || !(rq.inv < 1e30f) || (__float_as_uint(rq.scale) & 0x7fffffu) == 0x7fffffu;
  return rq;
}

constexpr float kRoundMagic = 12582912.0f;   // 1.5 * 2^23

// Word whose low byte is clamp(rint(v / scale)), by the library's IEEE division.
__device__ __forceinline__ uint32_t quant_word_exact(float v, float scale) {
  const float r = fminf(fmaxf(__fdiv_rn(v, scale), -127.f), 127.f);
  return __float_as_uint(__fadd_rn(r, kRoundMagic));
}

__device__ __forceinline__ uint32_t pack4_words(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

__device__ __forceinline__ uint2 quant8(const float (&v)[8], const RowQuant& rq) {
  if (!(rq.scale > 0.f)) return make_uint2(0u, 0u);
  uint32_t w[8];
  if (!rq.exact) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q0 = __fmul_rn(v[i], rq.inv);
      const float r = __fmaf_rn(-q0, rq.scale, v[i]);
      const float q1 = __fmaf_rn(r, rq.inv, q0);
      w[i] = __float_as_uint(__fadd_rn(q1, kRoundMagic));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = quant_word_exact(v[i], rq.scale);
  }
  uint2 o;
  o.x = pack4_words(w[0], w[1], w[2], w[3]);
  o.y = pack4_words(w[4], w[5], w[6], w[7]);
  return o;
}

// Four values -> four int8 in one word; the arithmetic of quant8.
__device__ __forceinline__ uint32_t quant4(const float (&v)[4], const RowQuant& rq) {
  if (!(rq.scale > 0.f)) return 0u;
  uint32_t w[4];
  if (!rq.exact) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float q0 = __fmul_rn(v[i], rq.inv);
      const float r = __fmaf_rn(-q0, rq.scale, v[i]);
      const float q1 = __fmaf_rn(r, rq.inv, q0);
      w[i] = __float_as_uint(__fadd_rn(q1, kRoundMagic));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = quant_word_exact(v[i], rq.scale);
  }
  return pack4_words(w[0], w[1], w[2], w[3]);
}

// max |x| over the 8 packed 16-bit elements of a raw chunk, without unpacking
__device__ __forceinline__ float raw_amax(const Raw8<__nv_bfloat16>& raw) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw.r);
  __nv_bfloat162 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
  return fmaxf(__low2float(m), __high2float(m));
}
__device__ __forceinline__ float raw_amax(const Raw8<__half>& raw) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw.r);
  __half2 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
  return fmaxf(__low2float(m), __high2float(m));
}
__device__ __forceinline__ float raw_amax(const Raw8<float>& raw) {
  return fmaxf(fmaxf(fmaxf(fabsf(raw.a.x), fabsf(raw.a.y)), fmaxf(fabsf(raw.a.z), fabsf(raw.a.w))),
               fmaxf(fmaxf(fabsf(raw.b.x), fabsf(raw.b.y)), fmaxf(fabsf(raw.b.z), fabsf(raw.b.w))));
}

// Copies one row of nvec 16-byte vectors with the CTA, eight loads in flight per thread before the stores.
template <int THREADS>
__device__ __forceinline__ void copy_row16(uint4* __restrict__ dst, const uint4* __restrict__ src, int nvec) {
  for (int v = threadIdx.x; v < nvec; v += 8 * THREADS) {
    uint4 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v + i * THREADS < nvec) t[i] = src[v + i * THREADS];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v + i * THREADS < nvec) __stcs(dst + v + i * THREADS, t[i]);   // streamed: keep the gathered source rows in L2
  }
}

// ---- rows -> group lookup for row kernels that follow a grouped GEMM ----
// Row ends of the groups in shared memory, computed once per CTA by its first warp (followed by a CTA barrier):
// the inclusive prefix of per-group counts, or the list itself when it already holds cumulative ends.
constexpr int kMaxDsqGroups = 4096;
__device__ __forceinline__ void group_ends_to_smem(const int64_t* __restrict__ list, int cumulative, int num_groups,
                                                   int* s_end) {
  if (threadIdx.x < 32) {   // one warp scans 32 groups per step
    const int lane = threadIdx.x;
    long long run = 0;
    for (int g0 = 0; g0 < num_groups; g0 += 32) {
      const int g = g0 + lane;
      long long c = g < num_groups ? list[g] : 0;
      if (c < 0) c = 0;
      if (cumulative) {
        if (g < num_groups) s_end[g] = static_cast<int>(min(c, 2147483647LL));
        continue;
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const long long t = __shfl_up_sync(0xffffffffu, c, o);
        if (lane >= o) c += t;
      }
      if (g < num_groups) s_end[g] = static_cast<int>(min(run + c, 2147483647LL));
      run += __shfl_sync(0xffffffffu, c, 31);
    }
  }
  __syncthreads();
}

// First group whose end is > row, or -1 when the row lies past every group.
__device__ __forceinline__ int group_of_row(const int* s_end, int num_groups, int64_t row) {
  if (num_groups == 0 || row >= s_end[num_groups - 1]) return -1;
  int lo = 0, hi = num_groups - 1;   // invariant: s_end[hi] > row
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (s_end[mid] > row) hi = mid; else lo = mid + 1;
  }
  return lo;
}

}  // namespace tab
