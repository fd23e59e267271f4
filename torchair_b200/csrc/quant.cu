// Per-row dynamic int8 quantisation (npu_dynamic_quant), SwiGLU (npu_swiglu) and the standalone
// dequant + SwiGLU + requant (npu_dequant_swiglu_quant).  All are HBM-bound row kernels: one CTA per row
// (64, 128 or 256 threads, picked so that a thread owns a few 16-byte chunks), the row kept in registers in its
// raw form between the amax pass and the store pass, many small CTAs per SM so that loads of one row overlap the
// reduction and stores of others.
#include "row_pipe.cuh"
#include "tab_common.cuh"

namespace tab {

// Status word of the staged row kernels on this device: 0, or 1 after a bulk-copy wait ran out (tab_quant_status).
__device__ int g_quant_status = 0;

constexpr int kMaxChunks = 8;  // chunks of 8 elements a thread keeps in registers; longer rows re-read their tail

// ---- staged form: rows of 1 KB .. 48 KB stream through a ring of shared-memory stages (row_pipe.cuh) ----------------
// One CTA barrier per row: the warps publish their maxima (double-buffered by row parity), every thread then reduces the
// eight values and derives the row's scale itself (a handful of instructions, see make_row_quant_fast); the stage of the
// previous row is refilled right after that barrier, when every thread is provably done with it.
constexpr int kRowStages = 3;
constexpr int kRowThreads = 256;
constexpr size_t kRowSmemBudget = 200 * 1024;   // per SM, for the rings of all resident CTAs

// amax / 127 and its reciprocal without the library's checked division: q = RN(amax / 127) by one correction step from
// the correctly rounded reciprocal of 127 (exact for every amax whose quotient and remainder are normal), inv by
// rcp_rn_normal.  Rows outside the safe range, and scales whose significand is all ones, take make_row_quant.
__device__ __forceinline__ RowQuant make_row_quant_fast(float amax) {
  if (!(amax > 1e-24f && amax < 1e30f)) return make_row_quant(amax);
  constexpr float kInv127 = 0x1.020408p-7f;    // RN(1 / 127)
  const float q0 = __fmul_rn(amax, kInv127);
  const float r = __fmaf_rn(-127.0f, q0, amax);
  RowQuant rq;
  rq.scale = __fmaf_rn(r, kInv127, q0);
  rq.inv = rcp_rn_normal(rq.scale);
  rq.exact = (__float_as_uint(rq.scale) & 0x7fffffu) == 0x7fffffu;
  return rq;
}

// Maximum over the CTA with one barrier; `red` is this row's buffer of one float per warp.
__device__ __forceinline__ float cta_max_once(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  const float4 a = *reinterpret_cast<const float4*>(red), b = *reinterpret_cast<const float4*>(red + 4);
  return fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
}

// Waits for ring slot k unless an earlier wait of this CTA already ran out; a wait that runs out is recorded.
template <int STAGES>
__device__ __forceinline__ void ring_wait_or_flag(const RowRing<STAGES>& ring, int k, volatile int* s_fail) {
  if (*s_fail == 0 && !ring.wait(k)) {
    *s_fail = 1;
    atomicCAS(&g_quant_status, 0, 1);
  }
}

// x [rows, cols] -> y int8, scale fp32; same arithmetic as dynamic_quant_kernel.  cols % 8 == 0, row bytes % 16 == 0.
template <typename T, bool kSmooth>
__global__ void __launch_bounds__(kRowThreads) dynamic_quant_staged_kernel(const T* __restrict__ x, const T* __restrict__ smooth,
                                                                          int64_t rows, int cols, int8_t* __restrict__ y,
                                                                          float* __restrict__ scale) {
  static_assert(kRowThreads == 256, "cta_max_once reads eight warp maxima");
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ uint64_t bars[kRowStages];
  __shared__ __align__(16) float red[2][kRowThreads / 32];
  __shared__ int s_fail;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
  RowRing<kRowStages> ring(ring_mem, bars, row_bytes, row_bytes);
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int64_t first = blockIdx.x, stride = gridDim.x;
  if (threadIdx.x == 0)
    for (int k = 0; k < kRowStages; ++k)
      if (first + k * stride < rows) ring.issue(k, x + (first + k * stride) * cols);
  const int nchunk = cols >> 3;
  auto value = [&](const T* sr, int ch, float (&v)[8]) {
    Raw8<T> raw;
    raw.load(sr + ch * 8);
    raw.unpack(v);
    if constexpr (kSmooth) {
      float sm[8];
      Elem<T>::load8(smooth + ch * 8, sm);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], sm[i]);
    }
  };
  int k = 0;
  for (int64_t row = first; row < rows; row += stride, ++k) {
    ring_wait_or_flag(ring, k, &s_fail);
    const T* sr = reinterpret_cast<const T*>(ring_mem + ring.stage_offset(k));
    float amax = 0.f;
    if constexpr (!kSmooth) {
#pragma unroll 4
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) {
        Raw8<T> raw;
        raw.load(sr + ch * 8);
        amax = fmaxf(amax, raw_amax(raw));
      }
    } else {
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) {
        float v[8];
        value(sr, ch, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
    }
    amax = cta_max_once(amax, red[k & 1]);
    // every thread has left the previous row behind: its stage takes the row kRowStages - 1 ahead of this one
    if (threadIdx.x == 0 && k >= 1 && row + (kRowStages - 1) * stride < rows)
      ring.issue(k - 1 + kRowStages, x + (row + (kRowStages - 1) * stride) * cols);
    const RowQuant sc = make_row_quant_fast(amax);
    if (threadIdx.x == 0) scale[row] = sc.scale;
    int8_t* yr = y + row * cols;
    if (sc.scale > 0.f && !sc.exact) {
      // the common case, free of per-element branches: four full-rate instructions per element
      const float inv = sc.inv, scl = sc.scale;
#pragma unroll 2
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) {
        float v[8];
        value(sr, ch, v);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float q0 = __fmul_rn(v[i], inv);
          const float r = __fmaf_rn(-q0, scl, v[i]);
          w[i] = __float_as_uint(__fadd_rn(__fmaf_rn(r, inv, q0), kRoundMagic));
        }
        __stcs(reinterpret_cast<uint2*>(yr + ch * 8), make_uint2(pack4_words(w[0], w[1], w[2], w[3]), pack4_words(w[4], w[5], w[6], w[7])));
      }
    } else {
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) {
        float v[8];
        value(sr, ch, v);
        __stcs(reinterpret_cast<uint2*>(yr + ch * 8), quant8(v, sc));
      }
    }
  }
}

// x int32 [rows, 2*half] -> y int8 [rows, half], scale [rows]; same arithmetic as dequant_swiglu_quant_kernel.  A thread
// takes four channels at a time: gate and up quadruples from the staged row, the fp32 SwiGLU values go back into the
// row's gate half in place (each thread re-reads only what it wrote), the second pass quantises them from there.
// half % 8 == 0.
// kQuads > 0: half == kQuads * 4 * kRowThreads exactly, the loops over a thread's quadruples unroll completely.
template <bool kLeft, bool kHasWs, int kQuads>
__global__ void __launch_bounds__(kRowThreads) dequant_swiglu_quant_staged_kernel(
    const int32_t* __restrict__ x, const float* __restrict__ wscale, int ws_groups, const float* __restrict__ ascale,
    const int64_t* __restrict__ group_index, int num_groups, int64_t rows, int half,
    int8_t* __restrict__ y, float* __restrict__ scale) {
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ uint64_t bars[kRowStages];
  __shared__ __align__(16) float red[2][kRowThreads / 32];
  __shared__ int s_fail;
  const uint32_t row_bytes = static_cast<uint32_t>(half) * 8u;
  int* s_end = reinterpret_cast<int*>(ring_mem + kRowStages * row_bytes);   // [num_groups], behind the ring
  if (group_index != nullptr) group_ends_to_smem(group_index, /*cumulative=*/0, num_groups, s_end);
  RowRing<kRowStages> ring(ring_mem, bars, row_bytes, row_bytes);
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int64_t first = blockIdx.x, stride = gridDim.x;
  if (threadIdx.x == 0)
    for (int k = 0; k < kRowStages; ++k)
      if (first + k * stride < rows) ring.issue(k, x + (first + k * stride) * 2 * half);
  const int nquad = half >> 2;
  int g = 0;       // group of the current row: rows only move forward, so the cursor does too
  int k = 0;
  for (int64_t row = first; row < rows; row += stride, ++k) {
    ring_wait_or_flag(ring, k, &s_fail);
    int32_t* sr = reinterpret_cast<int32_t*>(ring_mem + ring.stage_offset(k));
    if (group_index != nullptr)
      while (g < num_groups && s_end[g] <= row) ++g;
    const bool covered = group_index == nullptr || g < num_groups;      // uniform over the CTA
    const float as = (covered && ascale) ? ascale[row] : 1.0f;
    const float* ws = (kHasWs && covered) ? wscale + (ws_groups > 1 ? static_cast<int64_t>(g) * 2 * half : 0) : nullptr;
    float amax = 0.f;
    float keep[kQuads > 0 ? kQuads : 1][4];     // kQuads > 0: the thread's SwiGLU values stay in registers between the passes
    if (covered) {
#pragma unroll
      for (int it = 0; it < (kQuads > 0 ? kQuads : (nquad + kRowThreads - 1) / kRowThreads); ++it) {
        const int q = threadIdx.x + it * kRowThreads;
        if (kQuads == 0 && q >= nquad) break;
        const int4 l = *reinterpret_cast<const int4*>(sr + q * 4);
        const int4 r = *reinterpret_cast<const int4*>(sr + half + q * 4);
        float lv[4] = {__fmul_rn(__int2float_rn(l.x), as), __fmul_rn(__int2float_rn(l.y), as), __fmul_rn(__int2float_rn(l.z), as),
                       __fmul_rn(__int2float_rn(l.w), as)};
        float rv[4] = {__fmul_rn(__int2float_rn(r.x), as), __fmul_rn(__int2float_rn(r.y), as), __fmul_rn(__int2float_rn(r.z), as),
                       __fmul_rn(__int2float_rn(r.w), as)};
        if constexpr (kHasWs) {
          const float4 wl = __ldg(reinterpret_cast<const float4*>(ws + q * 4));
          const float4 wr = __ldg(reinterpret_cast<const float4*>(ws + half + q * 4));
          lv[0] = __fmul_rn(lv[0], wl.x); lv[1] = __fmul_rn(lv[1], wl.y); lv[2] = __fmul_rn(lv[2], wl.z); lv[3] = __fmul_rn(lv[3], wl.w);
          rv[0] = __fmul_rn(rv[0], wr.x); rv[1] = __fmul_rn(rv[1], wr.y); rv[2] = __fmul_rn(rv[2], wr.z); rv[3] = __fmul_rn(rv[3], wr.w);
        }
        float h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          h[i] = kLeft ? silu_mul(lv[i], rv[i]) : silu_mul(rv[i], lv[i]);
          amax = fmaxf(amax, fabsf(h[i]));
        }
        if constexpr (kQuads > 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) keep[it][i] = h[i];
        } else {
          *reinterpret_cast<float4*>(sr + q * 4) = make_float4(h[0], h[1], h[2], h[3]);   // in place over the gate quadruple
        }
      }
    }
    amax = cta_max_once(amax, red[k & 1]);
    if (threadIdx.x == 0 && k >= 1 && row + (kRowStages - 1) * stride < rows)
      ring.issue(k - 1 + kRowStages, x + (row + (kRowStages - 1) * stride) * 2 * half);
    int8_t* yr = y + row * half;
    if (!covered) {  // row outside every group
      for (int q = threadIdx.x; q < nquad; q += kRowThreads) *reinterpret_cast<uint32_t*>(yr + q * 4) = 0u;
      if (threadIdx.x == 0) scale[row] = 0.f;
      continue;
    }
    const RowQuant sc = make_row_quant_fast(amax);
    if (threadIdx.x == 0) scale[row] = sc.scale;
    const float* hr = reinterpret_cast<const float*>(sr);
    if (sc.scale > 0.f && !sc.exact) {
      const float inv = sc.inv, scl = sc.scale;
#pragma unroll
      for (int it = 0; it < (kQuads > 0 ? kQuads : (nquad + kRowThreads - 1) / kRowThreads); ++it) {
        const int q = threadIdx.x + it * kRowThreads;
        if (kQuads == 0 && q >= nquad) break;
        float v[4];
        if constexpr (kQuads > 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = keep[it][i];
        } else {
          const float4 a = *reinterpret_cast<const float4*>(hr + q * 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        }
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float q0 = __fmul_rn(v[i], inv);
          const float r = __fmaf_rn(-q0, scl, v[i]);
          w[i] = __float_as_uint(__fadd_rn(__fmaf_rn(r, inv, q0), kRoundMagic));
        }
        __stcs(reinterpret_cast<uint32_t*>(yr + q * 4), pack4_words(w[0], w[1], w[2], w[3]));
      }
    } else {
      for (int it = 0; it * kRowThreads + static_cast<int>(threadIdx.x) < nquad; ++it) {
        const int q = threadIdx.x + it * kRowThreads;
        float v[4];
        if constexpr (kQuads > 0) {
#pragma unroll
          for (int j = 0; j < kQuads; ++j)
            if (j == it) {
#pragma unroll
              for (int i = 0; i < 4; ++i) v[i] = keep[j][i];
            }
        } else {
          const float4 a = *reinterpret_cast<const float4*>(hr + q * 4);
          v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        }
        __stcs(reinterpret_cast<uint32_t*>(yr + q * 4), quant4(v, sc));
      }
    }
  }
}

// Persistent grid and ring size for a staged row kernel, or 0 when the rows do not suit it (tiny or too long for three
// stages): CTAs per SM by the shared-memory budget, at most 8.
static int staged_grid(int64_t rows, size_t row_bytes, size_t* smem_bytes) {
  if (row_bytes < 1024 || row_bytes % 16 != 0 || row_bytes * kRowStages > 192 * 1024) return 0;
  *smem_bytes = row_bytes * kRowStages;
  size_t per_sm = kRowSmemBudget / (*smem_bytes + 1024);
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  return grid_for(rows, static_cast<int>(per_sm));
}

// x [rows, cols] -> y int8, scale fp32.  cols % 8 == 0.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) dynamic_quant_kernel(const T* __restrict__ x, const T* __restrict__ smooth,
                                                               int64_t rows, int cols, int8_t* __restrict__ y,
                                                               float* __restrict__ scale) {
  __shared__ float red[THREADS / 32];
  const int nchunk = cols >> 3;
  auto value = [&](const Raw8<T>& raw, int ch, float (&v)[8]) {
    raw.unpack(v);
    if (smooth != nullptr) {
      float s[8];
      Elem<T>::load8(smooth + ch * 8, s);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], s[i]);
    }
  };
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    Raw8<T> raw[kMaxChunks];
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < nchunk) raw[c].load(xr + ch * 8);
    }
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < nchunk) {
        if (smooth == nullptr) {
          amax = fmaxf(amax, raw_amax(raw[c]));
        } else {
          float v[8];
          value(raw[c], ch, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        }
      }
    }
    for (int ch = threadIdx.x + kMaxChunks * THREADS; ch < nchunk; ch += THREADS) {
      Raw8<T> t;
      t.load(xr + ch * 8);
      float v[8];
      value(t, ch, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = cta_max<THREADS>(amax, red);
    const RowQuant sc = make_row_quant(amax);
    if (threadIdx.x == 0) scale[row] = sc.scale;
    int8_t* yr = y + row * cols;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < nchunk) {
        float v[8];
        value(raw[c], ch, v);
        __stcs(reinterpret_cast<uint2*>(yr + ch * 8), quant8(v, sc));
      }
    }
    for (int ch = threadIdx.x + kMaxChunks * THREADS; ch < nchunk; ch += THREADS) {
      Raw8<T> t;
      t.load(xr + ch * 8);   // still in L2
      float v[8];
      value(t, ch, v);
      *reinterpret_cast<uint2*>(yr + ch * 8) = quant8(v, sc);
    }
  }
}

// y[r, c] = silu(x[r, c]) * x[r, c + half]; one thread per 8 output elements.  A CTA of 256 threads covers
// 256 / tpr rows at a time with tpr threads per row (tpr = a power of two, at most 256, chosen by the host so that
// short rows still fill the CTA).  Pointers advance by a constant per row step: no multiply or division in the loop.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ x, int64_t rows, int half, int tpr_log2,
                                                     T* __restrict__ y) {
  const int chunks_per_row = half >> 3;
  const int tpr = 1 << tpr_log2;
  const int rows_per_cta = 256 >> tpr_log2;
  const int lane_in_row = threadIdx.x & (tpr - 1);
  const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta + (threadIdx.x >> tpr_log2);
  const int64_t row_step = static_cast<int64_t>(gridDim.x) * rows_per_cta;
  const T* xr = x + r0 * 2 * half;
  T* yr = y + r0 * half;
  const int64_t x_step = row_step * 2 * half, y_step = row_step * half;
  for (int64_t r = r0; r < rows; r += row_step, xr += x_step, yr += y_step) {
    for (int ch = lane_in_row; ch < chunks_per_row; ch += tpr) {
      float a[8], b[8], o[8];
      Elem<T>::load8(xr + ch * 8, a);
      Elem<T>::load8(xr + half + ch * 8, b);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = silu_mul(a[k], b[k]);
      Elem<T>::store8(yr + ch * 8, o);
    }
  }
}

// x int32 [rows, 2*half] -> y int8 [rows, half], scale [rows]; one CTA per row.
constexpr int kDsqChunks = 4;
template <int THREADS>
__global__ void __launch_bounds__(THREADS) dequant_swiglu_quant_kernel(
    const int32_t* __restrict__ x, const float* __restrict__ wscale, int ws_groups, const float* __restrict__ ascale,
    const int64_t* __restrict__ group_index, int num_groups, int activate_left, int64_t rows, int half,
    int8_t* __restrict__ y, float* __restrict__ scale) {
  __shared__ float red[THREADS / 32];
  extern __shared__ int s_end[];
  if (group_index != nullptr) group_ends_to_smem(group_index, /*cumulative=*/0, num_groups, s_end);
  const int nchunk = half >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int g = group_index != nullptr ? group_of_row(s_end, num_groups, row) : 0;   // uniform over the CTA
    int8_t* yr = y + row * half;
    if (g < 0) {  // row outside every group
      for (int ch = threadIdx.x; ch < nchunk; ch += THREADS) *reinterpret_cast<uint2*>(yr + ch * 8) = make_uint2(0, 0);
      if (threadIdx.x == 0) scale[row] = 0.f;
      continue;
    }
    const float as = ascale ? ascale[row] : 1.0f;
    const float* ws = wscale ? wscale + (ws_groups > 1 ? static_cast<int64_t>(g) * 2 * half : 0) : nullptr;
    const int32_t* xr = x + row * 2 * half;
    auto compute = [&](int ch, float (&o)[8]) {
      const int c = ch * 8;
      const int4 l0 = *reinterpret_cast<const int4*>(xr + c), l1 = *reinterpret_cast<const int4*>(xr + c + 4);
      const int4 r0 = *reinterpret_cast<const int4*>(xr + half + c), r1 = *reinterpret_cast<const int4*>(xr + half + c + 4);
      float l[8] = {__int2float_rn(l0.x), __int2float_rn(l0.y), __int2float_rn(l0.z), __int2float_rn(l0.w),
                    __int2float_rn(l1.x), __int2float_rn(l1.y), __int2float_rn(l1.z), __int2float_rn(l1.w)};
      float r[8] = {__int2float_rn(r0.x), __int2float_rn(r0.y), __int2float_rn(r0.z), __int2float_rn(r0.w),
                    __int2float_rn(r1.x), __int2float_rn(r1.y), __int2float_rn(r1.z), __int2float_rn(r1.w)};
      float wl[8], wr[8];
      if (ws) {
        Elem<float>::load8(ws + c, wl);
        Elem<float>::load8(ws + half + c, wr);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float lv = __fmul_rn(l[k], as), rv = __fmul_rn(r[k], as);
        if (ws) {
          lv = __fmul_rn(lv, wl[k]);
          rv = __fmul_rn(rv, wr[k]);
        }
        o[k] = silu_mul(activate_left ? lv : rv, activate_left ? rv : lv);   // one SwiGLU, operands picked first
      }
    };
    float h[kDsqChunks][8];
    float amax = 0.f;
#pragma unroll
    for (int cc = 0; cc < kDsqChunks; ++cc) {
      const int ch = threadIdx.x + cc * THREADS;
      if (ch < nchunk) {
        compute(ch, h[cc]);
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(h[cc][k]));
      }
    }
    for (int ch = threadIdx.x + kDsqChunks * THREADS; ch < nchunk; ch += THREADS) {
      float t[8];
      compute(ch, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(t[k]));
    }
    amax = cta_max<THREADS>(amax, red);
    const RowQuant sc = make_row_quant(amax);
    if (threadIdx.x == 0) scale[row] = sc.scale;
#pragma unroll
    for (int cc = 0; cc < kDsqChunks; ++cc) {
      const int ch = threadIdx.x + cc * THREADS;
      if (ch < nchunk) *reinterpret_cast<uint2*>(yr + ch * 8) = quant8(h[cc], sc);
    }
    for (int ch = threadIdx.x + kDsqChunks * THREADS; ch < nchunk; ch += THREADS) {
      float t[8];
      compute(ch, t);
      *reinterpret_cast<uint2*>(yr + ch * 8) = quant8(t, sc);
    }
  }
}

// Second phase of the fused gate_up GEMM: h fp32 [rows, cols] + row amax bits -> int8 + scale; rows at or past the
// rows covered by group_list are left untouched.
template <int THREADS>
__global__ void __launch_bounds__(THREADS) quant_from_f32_kernel(const float* __restrict__ h,
                                                                const uint32_t* __restrict__ amax_bits,
                                                                const int64_t* __restrict__ group_list,
                                                                int group_list_type, int num_groups, int64_t rows,
                                                                int cols, int8_t* __restrict__ y,
                                                                float* __restrict__ scale) {
  __shared__ long long s_valid;
  if (threadIdx.x < 32) {
    long long v = 0;
    if (group_list_type == 0) {
      v = num_groups > 0 ? group_list[num_groups - 1] : 0;
    } else {
      for (int g = threadIdx.x; g < num_groups; g += 32) v += group_list[g] > 0 ? group_list[g] : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    if (threadIdx.x == 0) s_valid = v;
  }
  __syncthreads();
  const int64_t valid = s_valid;
  const int nchunk = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int8_t* yr = y + row * cols;
    if (row >= valid) break;   // rows outside every group are not touched (they may be a large unused tail)
    const RowQuant sc = make_row_quant(__uint_as_float(amax_bits[row]));
    if (threadIdx.x == 0) scale[row] = sc.scale;
    const float* hr = h + row * cols;
    for (int ch0 = threadIdx.x; ch0 < nchunk; ch0 += 4 * THREADS) {
      float t[4][8];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (ch0 + i * THREADS < nchunk) Elem<float>::load8(hr + (ch0 + i * THREADS) * 8, t[i]);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (ch0 + i * THREADS < nchunk) *reinterpret_cast<uint2*>(yr + (ch0 + i * THREADS) * 8) = quant8(t[i], sc);
    }
  }
}

// CTAs per SM for a row kernel of THREADS threads (register-limited estimate), times the SM count.
static int row_grid(int64_t rows, int threads) { return grid_for(rows, threads >= 256 ? 5 : threads >= 128 ? 10 : 16); }

int launch_quant_from_f32(const float* h, const uint32_t* amax_bits, const int64_t* group_list,
                          int group_list_type, int num_groups, int64_t rows, int cols, int8_t* y,
                          float* scale, cudaStream_t st) {
  if (rows == 0) return TAB_OK;
  const int nchunk = cols / 8;
  if (nchunk <= 256)
    quant_from_f32_kernel<64><<<row_grid(rows, 64), 64, 0, st>>>(h, amax_bits, group_list, group_list_type, num_groups, rows, cols, y, scale);
  else
    quant_from_f32_kernel<256><<<row_grid(rows, 256), 256, 0, st>>>(h, amax_bits, group_list, group_list_type, num_groups, rows, cols, y, scale);
  return check_launch("quant_from_f32");
}

template <typename T>
static void launch_dynamic_quant(const void* x, const void* smooth, int64_t rows, int cols, int8_t* y, float* scale,
                                 cudaStream_t st) {
  const int nchunk = cols / 8;
  const T* xp = static_cast<const T*>(x);
  const T* sp = static_cast<const T*>(smooth);
  size_t smem = 0;
  const int sgrid = rows >= 64 ? staged_grid(rows, static_cast<size_t>(cols) * sizeof(T), &smem) : 0;
  if (sgrid > 0 && sp == nullptr &&
      cudaFuncSetAttribute(dynamic_quant_staged_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess) {
    dynamic_quant_staged_kernel<T, false><<<sgrid, kRowThreads, smem, st>>>(xp, sp, rows, cols, y, scale);
    return;
  }
  if (sgrid > 0 && sp != nullptr &&
      cudaFuncSetAttribute(dynamic_quant_staged_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess) {
    dynamic_quant_staged_kernel<T, true><<<sgrid, kRowThreads, smem, st>>>(xp, sp, rows, cols, y, scale);
    return;
  }
  if (nchunk <= 64 * kMaxChunks / 2)
    dynamic_quant_kernel<T, 64><<<grid_for(rows, 16), 64, 0, st>>>(xp, sp, rows, cols, y, scale);
  else if (nchunk <= 128 * kMaxChunks)
    dynamic_quant_kernel<T, 128><<<grid_for(rows, 8), 128, 0, st>>>(xp, sp, rows, cols, y, scale);
  else
    dynamic_quant_kernel<T, 256><<<grid_for(rows, 4), 256, 0, st>>>(xp, sp, rows, cols, y, scale);
}

}  // namespace tab

using namespace tab;

extern "C" int tab_dynamic_quant(const void* x, int x_dtype, const void* smooth, int64_t rows, int64_t cols,
                                 int8_t* y, float* scale, tab_stream_t stream) {
  if (rows < 0 || cols <= 0) return fail(TAB_ERR_BAD_ARG, "dynamic_quant: rows=%lld cols=%lld", (long long)rows, (long long)cols);
  if (rows == 0) return TAB_OK;
  if (!x || !y || !scale) return fail(TAB_ERR_BAD_ARG, "dynamic_quant: null pointer");
  if (cols % 16 != 0 || cols > (1 << 24)) return fail(TAB_ERR_ALIGNMENT, "dynamic_quant: cols=%lld must be a multiple of 16", (long long)cols);
  if (!aligned16(x) || !aligned16(y) || (smooth && !aligned16(smooth))) return fail(TAB_ERR_ALIGNMENT, "dynamic_quant: pointers must be 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  switch (x_dtype) {
    case TAB_BF16: launch_dynamic_quant<__nv_bfloat16>(x, smooth, rows, (int)cols, y, scale, st); break;
    case TAB_F16: launch_dynamic_quant<__half>(x, smooth, rows, (int)cols, y, scale, st); break;
    case TAB_F32: launch_dynamic_quant<float>(x, smooth, rows, (int)cols, y, scale, st); break;
    default: return fail(TAB_ERR_UNSUPPORTED, "dynamic_quant: input dtype %d (want 5, 6 or 15)", x_dtype);
  }
  return check_launch("dynamic_quant");
}

extern "C" int tab_swiglu(const void* x, int dtype, int64_t rows, int64_t cols, void* y, tab_stream_t stream) {
  if (rows < 0 || cols <= 0 || (cols & 1)) return fail(TAB_ERR_BAD_ARG, "swiglu: rows=%lld cols=%lld (cols must be even)", (long long)rows, (long long)cols);
  if (rows == 0) return TAB_OK;
  if (!x || !y) return fail(TAB_ERR_BAD_ARG, "swiglu: null pointer");
  const int64_t half = cols / 2;
  if (half % 8 != 0 || !aligned16(x) || !aligned16(y)) return fail(TAB_ERR_ALIGNMENT, "swiglu: cols/2=%lld must be a multiple of 8 and pointers 16-byte aligned", (long long)half);
  cudaStream_t st = as_stream(stream);
  const int64_t chunks = half / 8;
  int tpr_log2 = 0;
  while ((1 << tpr_log2) < chunks && tpr_log2 < 8) ++tpr_log2;
  const int64_t ctas = (rows + (256 >> tpr_log2) - 1) / (256 >> tpr_log2);
  const int grid = grid_for(ctas, 8);
  switch (dtype) {
    case TAB_BF16:
      swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, (int)half, tpr_log2, static_cast<__nv_bfloat16*>(y));
      break;
    case TAB_F16:
      swiglu_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), rows, (int)half, tpr_log2, static_cast<__half*>(y));
      break;
    case TAB_F32:
      swiglu_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), rows, (int)half, tpr_log2, static_cast<float*>(y));
      break;
    default:
      return fail(TAB_ERR_UNSUPPORTED, "swiglu: dtype %d (want 5, 6 or 15)", dtype);
  }
  return check_launch("swiglu");
}

extern "C" int tab_dequant_swiglu_quant(const int32_t* x, const float* weight_scale, int64_t ws_groups,
                                        const float* activation_scale, const int64_t* group_index,
                                        int64_t num_groups, int activate_left, int64_t rows, int64_t cols,
                                        int8_t* y, float* scale, tab_stream_t stream) {
  if (rows < 0 || cols <= 0 || (cols & 1)) return fail(TAB_ERR_BAD_ARG, "dequant_swiglu_quant: rows=%lld cols=%lld (cols must be even)", (long long)rows, (long long)cols);
  if (rows == 0) return TAB_OK;
  if (!x || !y || !scale) return fail(TAB_ERR_BAD_ARG, "dequant_swiglu_quant: null pointer");
  const int64_t half = cols / 2;
  if (half % 8 != 0 || !aligned16(x) || !aligned16(y) || (weight_scale && !aligned16(weight_scale)))
    return fail(TAB_ERR_ALIGNMENT, "dequant_swiglu_quant: cols/2=%lld must be a multiple of 8 and pointers 16-byte aligned", (long long)half);
  if (weight_scale && ws_groups > 1 && (!group_index || num_groups != ws_groups))
    return fail(TAB_ERR_BAD_ARG, "dequant_swiglu_quant: per-group weight_scale [%lld, cols] needs group_index of the same length (got %lld)", (long long)ws_groups, (long long)num_groups);
  if (num_groups > kMaxDsqGroups) return fail(TAB_ERR_UNSUPPORTED, "dequant_swiglu_quant: more than %d groups", kMaxDsqGroups);
  cudaStream_t st = as_stream(stream);
  const int nchunk = (int)(half / 8);
  size_t ring_bytes = 0;
  int sgrid = rows >= 64 ? staged_grid(rows, static_cast<size_t>(half) * 8, &ring_bytes) : 0;
  ring_bytes += static_cast<size_t>(num_groups) * sizeof(int);
  if (ring_bytes > 200 * 1024) sgrid = 0;
  if (sgrid > 0) {
#define TAB_DSQ(L, W, Q)                                                                                                         \
  if (cudaFuncSetAttribute(dequant_swiglu_quant_staged_kernel<L, W, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                           static_cast<int>(ring_bytes)) == cudaSuccess) {                                                      \
    dequant_swiglu_quant_staged_kernel<L, W, Q><<<sgrid, kRowThreads, ring_bytes, st>>>(x, weight_scale, (int)ws_groups, activation_scale, \
                                                                                       group_index, (int)num_groups, rows, (int)half, y, scale); \
    return check_launch("dequant_swiglu_quant");                                                                               \
  }
#define TAB_DSQ_Q(L, W)                                                       \
  if (half == 2 * 4 * kRowThreads) { TAB_DSQ(L, W, 2) }                        \
  else if (half == 4 * kRowThreads) { TAB_DSQ(L, W, 1) }                       \
  else { TAB_DSQ(L, W, 0) }
    if (activate_left) {
      if (weight_scale) { TAB_DSQ_Q(true, true) } else { TAB_DSQ_Q(true, false) }
    } else {
      if (weight_scale) { TAB_DSQ_Q(false, true) } else { TAB_DSQ_Q(false, false) }
    }
#undef TAB_DSQ_Q
#undef TAB_DSQ
  }
  const size_t smem = group_index ? static_cast<size_t>(num_groups) * sizeof(int) : 0;
  if (nchunk <= 64 * kDsqChunks / 2)
    dequant_swiglu_quant_kernel<64><<<row_grid(rows, 64), 64, smem, st>>>(x, weight_scale, (int)ws_groups, activation_scale, group_index, (int)num_groups, activate_left, rows, (int)half, y, scale);
  else if (nchunk <= 128 * kDsqChunks / 2)
    dequant_swiglu_quant_kernel<128><<<row_grid(rows, 128), 128, smem, st>>>(x, weight_scale, (int)ws_groups, activation_scale, group_index, (int)num_groups, activate_left, rows, (int)half, y, scale);
  else
    dequant_swiglu_quant_kernel<256><<<row_grid(rows, 256), 256, smem, st>>>(x, weight_scale, (int)ws_groups, activation_scale, group_index, (int)num_groups, activate_left, rows, (int)half, y, scale);
  return check_launch("dequant_swiglu_quant");
}

extern "C" int tab_quant_status(int* status_host, tab_stream_t stream) {
  if (!status_host) return fail(TAB_ERR_BAD_ARG, "quant_status: null pointer");
  cudaError_t e = cudaStreamSynchronize(as_stream(stream));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(status_host, g_quant_status, sizeof(int));
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "quant_status: %s", cudaGetErrorString(e));
  if (*status_host != 0) return fail(TAB_ERR_TIMEOUT, "row kernels: a bulk-copy wait gave up (status %d)", *status_host);
  return TAB_OK;
}

// Exhaustive self-test of rcp_rn_normal and of make_row_quant_fast against the library's IEEE reciprocal and division:
// all 2^23 significands at one exponent.
namespace tab {
__global__ void __launch_bounds__(256) selftest_reciprocal_kernel(int exponent, unsigned long long* mismatches) {
  const unsigned m = blockIdx.x * 256u + threadIdx.x;
  const float d = __uint_as_float((static_cast<unsigned>(127 + exponent) << 23) | m);
  if (rcp_rn_normal(d) != __frcp_rn(d)) atomicAdd(mismatches, 1ull);
  const RowQuant fast = make_row_quant_fast(d), lib = make_row_quant(d);        // d as a row maximum: amax / 127 and its reciprocal
  if (fast.scale != lib.scale || fast.inv != lib.inv) atomicAdd(mismatches, 1ull);
}
}  // namespace tab

extern "C" int tab_selftest_reciprocal(int exponent, unsigned long long* mismatches, tab_stream_t stream) {
  if (!mismatches || exponent < -100 || exponent > 120) return fail(TAB_ERR_BAD_ARG, "selftest_reciprocal: exponent %d (want -100..120)", exponent);
  selftest_reciprocal_kernel<<<(1 << 23) / 256, 256, 0, as_stream(stream)>>>(exponent, mismatches);
  return check_launch("selftest_reciprocal");
}
