// Per-row dynamic int8 quantisation (npu_dynamic_quant), SwiGLU (npu_swiglu) and the standalone
// dequant + SwiGLU + requant (npu_dequant_swiglu_quant).  All three are HBM-bound row kernels: one CTA
// per row, 16-byte loads, the row kept in registers between the amax pass and the store pass.
#include "tab_common.cuh"

namespace tab {

constexpr int kRowThreads = 256;
constexpr int kMaxChunks = 8;  // 8 elements each: rows up to 256*8*8 = 16384 columns stay in registers

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  r = warp_max(r);
  __syncthreads();
  return r;
}

__device__ __forceinline__ void store8_i8(int8_t* p, const float (&v)[8], float scale) {
  uint2 o;
  o.x = pack4_i8(quant_i8(v[0], scale), quant_i8(v[1], scale), quant_i8(v[2], scale), quant_i8(v[3], scale));
  o.y = pack4_i8(quant_i8(v[4], scale), quant_i8(v[5], scale), quant_i8(v[6], scale), quant_i8(v[7], scale));
  *reinterpret_cast<uint2*>(p) = o;
}

// x [rows, cols] -> y int8, scale fp32.  cols % 8 == 0.  Rows with more than kMaxChunks*kRowThreads
// chunks re-read the tail from global memory (it is still in L2) in the store pass.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) dynamic_quant_kernel(const T* __restrict__ x,
                                                                   const T* __restrict__ smooth,
                                                                   int64_t rows, int cols,
                                                                   int8_t* __restrict__ y,
                                                                   float* __restrict__ scale) {
  __shared__ float red[32];
  const int nchunk = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    float v[kMaxChunks][8];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      const int ch = threadIdx.x + c * kRowThreads;
      if (ch < nchunk) {
        Elem<T>::load8(xr + ch * 8, v[c]);
        if (smooth != nullptr) {
          float s[8];
          Elem<T>::load8(smooth + ch * 8, s);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c][i] = __fmul_rn(v[c][i], s[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[c][i]));
      }
    }
    for (int ch = threadIdx.x + kMaxChunks * kRowThreads; ch < nchunk; ch += kRowThreads) {
      float t[8];
      Elem<T>::load8(xr + ch * 8, t);
      if (smooth != nullptr) {
        float s[8];
        Elem<T>::load8(smooth + ch * 8, s);
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = __fmul_rn(t[i], s[i]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(t[i]));
    }
    amax = block_max(amax, red);
    const float sc = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) scale[row] = sc;
    int8_t* yr = y + row * cols;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
      const int ch = threadIdx.x + c * kRowThreads;
      if (ch < nchunk) store8_i8(yr + ch * 8, v[c], sc);
    }
    for (int ch = threadIdx.x + kMaxChunks * kRowThreads; ch < nchunk; ch += kRowThreads) {
      float t[8];
      Elem<T>::load8(xr + ch * 8, t);
      if (smooth != nullptr) {
        float s[8];
        Elem<T>::load8(smooth + ch * 8, s);
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = __fmul_rn(t[i], s[i]);
      }
      store8_i8(yr + ch * 8, t, sc);
    }
  }
}

// y[r, c] = silu(x[r, c]) * x[r, c + half]; one thread per 8 output elements, grid-stride.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ x, int64_t rows, int half,
                                                     T* __restrict__ y) {
  const int chunks_per_row = half >> 3;
  const int64_t total = rows * chunks_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / chunks_per_row;
    const int c = static_cast<int>(i - r * chunks_per_row) * 8;
    float a[8], b[8], o[8];
    Elem<T>::load8(x + r * 2 * half + c, a);
    Elem<T>::load8(x + r * 2 * half + half + c, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = silu_mul(a[k], b[k]);
    Elem<T>::store8(y + r * half + c, o);
  }
}

// Finds the group of `row` from per-group counts; returns -1 past their sum.  Warp-cooperative would be
// overkill: groups <= 1024 and the scan runs once per CTA-row out of L1/L2.
__device__ __forceinline__ int group_of_row(const int64_t* __restrict__ counts, int num_groups, int64_t row) {
  int64_t end = 0;
  for (int g = 0; g < num_groups; ++g) {
    int64_t c = counts[g];
    end += c > 0 ? c : 0;
    if (row < end) return g;
  }
  return -1;
}

// x int32 [rows, 2*half] -> y int8 [rows, half], scale [rows]; one CTA per row.
constexpr int kDsqChunks = 4;  // half up to 256*8*4 = 8192 kept in registers
__global__ void __launch_bounds__(kRowThreads) dequant_swiglu_quant_kernel(
    const int32_t* __restrict__ x, const float* __restrict__ wscale, int ws_groups,
    const float* __restrict__ ascale, const int64_t* __restrict__ group_index, int num_groups,
    int activate_left, int64_t rows, int half, int8_t* __restrict__ y, float* __restrict__ scale) {
  __shared__ float red[32];
  __shared__ int s_group;
  const int nchunk = half >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    if (threadIdx.x == 0) s_group = group_index ? group_of_row(group_index, num_groups, row) : 0;
    __syncthreads();
    const int g = s_group;
    int8_t* yr = y + row * half;
    if (g < 0) {  // row outside every group
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) *reinterpret_cast<uint2*>(yr + ch * 8) = make_uint2(0, 0);
      if (threadIdx.x == 0) scale[row] = 0.f;
      __syncthreads();
      continue;
    }
    const float as = ascale ? ascale[row] : 1.0f;
    const float* ws = wscale ? wscale + (ws_groups > 1 ? static_cast<int64_t>(g) * 2 * half : 0) : nullptr;
    const int32_t* xr = x + row * 2 * half;
    float h[kDsqChunks][8];
    float amax = 0.f;
    auto compute = [&](int ch, float (&o)[8]) {
      const int c = ch * 8;
      int4 l0 = *reinterpret_cast<const int4*>(xr + c), l1 = *reinterpret_cast<const int4*>(xr + c + 4);
      int4 r0 = *reinterpret_cast<const int4*>(xr + half + c), r1 = *reinterpret_cast<const int4*>(xr + half + c + 4);
      const int li[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
      const int ri[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float l = __fmul_rn(__int2float_rn(li[k]), as);
        float r = __fmul_rn(__int2float_rn(ri[k]), as);
        if (ws) {
          l = __fmul_rn(l, ws[c + k]);
          r = __fmul_rn(r, ws[half + c + k]);
        }
        o[k] = activate_left ? silu_mul(l, r) : silu_mul(r, l);
      }
    };
#pragma unroll
    for (int cc = 0; cc < kDsqChunks; ++cc) {
      const int ch = threadIdx.x + cc * kRowThreads;
      if (ch < nchunk) {
        compute(ch, h[cc]);
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(h[cc][k]));
      }
    }
    for (int ch = threadIdx.x + kDsqChunks * kRowThreads; ch < nchunk; ch += kRowThreads) {
      float t[8];
      compute(ch, t);
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(t[k]));
    }
    amax = block_max(amax, red);
    const float sc = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) scale[row] = sc;
#pragma unroll
    for (int cc = 0; cc < kDsqChunks; ++cc) {
      const int ch = threadIdx.x + cc * kRowThreads;
      if (ch < nchunk) store8_i8(yr + ch * 8, h[cc], sc);
    }
    for (int ch = threadIdx.x + kDsqChunks * kRowThreads; ch < nchunk; ch += kRowThreads) {
      float t[8];
      compute(ch, t);
      store8_i8(yr + ch * 8, t, sc);
    }
  }
}

// Second phase of the fused gate_up GEMM: h fp32 [rows, cols] + row amax bits -> int8 + scale; rows at or
// past *valid_rows give zeros.  Also used nowhere else; lives here with the other row quantisers.
__global__ void __launch_bounds__(kRowThreads) quant_from_f32_kernel(const float* __restrict__ h,
                                                                    const uint32_t* __restrict__ amax_bits,
                                                                    const int64_t* __restrict__ group_list,
                                                                    int group_list_type, int num_groups,
                                                                    int64_t rows, int cols,
                                                                    int8_t* __restrict__ y,
                                                                    float* __restrict__ scale) {
  __shared__ int64_t s_valid;
  if (threadIdx.x == 0) {
    int64_t v = 0;
    if (group_list_type == 0) {
      v = num_groups > 0 ? group_list[num_groups - 1] : 0;
    } else {
      for (int g = 0; g < num_groups; ++g) v += group_list[g] > 0 ? group_list[g] : 0;
    }
    s_valid = v;
  }
  __syncthreads();
  const int64_t valid = s_valid;
  const int nchunk = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int8_t* yr = y + row * cols;
    if (row >= valid) {
      for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) *reinterpret_cast<uint2*>(yr + ch * 8) = make_uint2(0, 0);
      if (threadIdx.x == 0) scale[row] = 0.f;
      continue;
    }
    const float sc = __fdiv_rn(__uint_as_float(amax_bits[row]), 127.0f);
    if (threadIdx.x == 0) scale[row] = sc;
    const float* hr = h + row * cols;
    for (int ch = threadIdx.x; ch < nchunk; ch += kRowThreads) {
      float t[8];
      Elem<float>::load8(hr + ch * 8, t);
      store8_i8(yr + ch * 8, t, sc);
    }
  }
}

int launch_quant_from_f32(const float* h, const uint32_t* amax_bits, const int64_t* group_list,
                          int group_list_type, int num_groups, int64_t rows, int cols, int8_t* y,
                          float* scale, cudaStream_t st) {
  if (rows == 0) return TAB_OK;
  quant_from_f32_kernel<<<grid_for(rows, 8), kRowThreads, 0, st>>>(h, amax_bits, group_list, group_list_type,
                                                                   num_groups, rows, cols, y, scale);
  return check_launch("quant_from_f32");
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
  const int grid = grid_for(rows, 8);
  switch (x_dtype) {
    case TAB_BF16:
      dynamic_quant_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(smooth), rows, (int)cols, y, scale);
      break;
    case TAB_F16:
      dynamic_quant_kernel<__half><<<grid, kRowThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(smooth), rows, (int)cols, y, scale);
      break;
    case TAB_F32:
      dynamic_quant_kernel<float><<<grid, kRowThreads, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(smooth), rows, (int)cols, y, scale);
      break;
    default:
      return fail(TAB_ERR_UNSUPPORTED, "dynamic_quant: input dtype %d (want 5, 6 or 15)", x_dtype);
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
  const int64_t work = rows * (half / 8);
  const int grid = grid_for((work + 255) / 256, 8);
  switch (dtype) {
    case TAB_BF16:
      swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, (int)half, static_cast<__nv_bfloat16*>(y));
      break;
    case TAB_F16:
      swiglu_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), rows, (int)half, static_cast<__half*>(y));
      break;
    case TAB_F32:
      swiglu_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), rows, (int)half, static_cast<float*>(y));
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
  if (half % 8 != 0 || !aligned16(x) || !aligned16(y)) return fail(TAB_ERR_ALIGNMENT, "dequant_swiglu_quant: cols/2=%lld must be a multiple of 8 and pointers 16-byte aligned", (long long)half);
  if (weight_scale && ws_groups > 1 && (!group_index || num_groups != ws_groups))
    return fail(TAB_ERR_BAD_ARG, "dequant_swiglu_quant: per-group weight_scale [%lld, cols] needs group_index of the same length (got %lld)", (long long)ws_groups, (long long)num_groups);
  if (num_groups > 4096) return fail(TAB_ERR_UNSUPPORTED, "dequant_swiglu_quant: more than 4096 groups");
  dequant_swiglu_quant_kernel<<<grid_for(rows, 8), kRowThreads, 0, as_stream(stream)>>>(
      x, weight_scale, (int)ws_groups, activation_scale, group_index, (int)num_groups, activate_left, rows, (int)half, y, scale);
  return check_launch("dequant_swiglu_quant");
}
