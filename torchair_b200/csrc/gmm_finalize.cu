// npu_grouped_matmul_finalize_routing: the down-projection grouped GEMM followed by the weighted scatter-add that
// folds the K expert rows of a token back into one fp32 row.  Three launches on the caller's stream:
//   1. the tcgen05 grouped GEMM with raw int32 accumulators into the workspace,
//   2. an init pass that zeroes y and places the (weighted) shared-expert rows,
//   3. a row kernel that dequantises each accumulator row, scales it by its logit and adds it into
//      y[row_index[row]] with 16-byte vector reductions.
// The additions of one output row arrive in no fixed order, so y is reproducible only up to fp32 summation order.
#include "tab_common.cuh"

namespace tab {

constexpr int kFinThreads = 256;

// y fp32 [out_rows, N] = 0, except rows [shared_offset, shared_offset + shared_rows) = weight * shared (bf16).
__global__ void __launch_bounds__(kFinThreads) finalize_init_kernel(const __nv_bfloat16* __restrict__ shared,
                                                                    int64_t shared_rows, int64_t shared_offset,
                                                                    float weight, int64_t out_rows, int N,
                                                                    float* __restrict__ y) {
  const int nchunk = N >> 2;
  for (int64_t row = blockIdx.x; row < out_rows; row += gridDim.x) {
    float4* yr = reinterpret_cast<float4*>(y + row * N);
    const int64_t s = row - shared_offset;
    if (shared != nullptr && s >= 0 && s < shared_rows) {
      const uint2* sr = reinterpret_cast<const uint2*>(shared + s * N);
      for (int c = threadIdx.x; c < nchunk; c += kFinThreads) {
        const uint2 raw = sr[c];
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        yr[c] = make_float4(__fmul_rn(a.x, weight), __fmul_rn(a.y, weight), __fmul_rn(b.x, weight), __fmul_rn(b.y, weight));
      }
    } else {
      for (int c = threadIdx.x; c < nchunk; c += kFinThreads) yr[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// acc int32 [rows, N] -> y[row_index[row], :] += logit[row] * ((float(acc) * tok_scale[row]) * w_scale[g, :] + bias[g, :]).
// One CTA per row; rows past the last group, and rows whose index is outside [0, out_rows), add nothing.
template <typename IDX>
__global__ void __launch_bounds__(kFinThreads) finalize_scatter_kernel(
    const int32_t* __restrict__ acc, const float* __restrict__ w_scale, const __nv_bfloat16* __restrict__ bias,
    const float* __restrict__ tok_scale, const int64_t* __restrict__ group_list, int cumulative, int num_groups,
    const float* __restrict__ logit, const IDX* __restrict__ row_index, int64_t rows, int N, int64_t out_rows,
    float* __restrict__ y) {
  extern __shared__ int s_end[];
  group_ends_to_smem(group_list, cumulative, num_groups, s_end);
  const int nchunk = N >> 2;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int g = group_of_row(s_end, num_groups, row);   // uniform over the CTA
    if (g < 0) break;                                      // group ends are monotone: every later row is outside too
    const int64_t dst = static_cast<int64_t>(row_index[row]);
    if (dst < 0 || dst >= out_rows) continue;
    const float ts = tok_scale ? tok_scale[row] : 1.0f;
    const float lg = logit ? logit[row] : 1.0f;
    const int4* ar = reinterpret_cast<const int4*>(acc + row * N);
    const float4* wr = w_scale ? reinterpret_cast<const float4*>(w_scale + static_cast<int64_t>(g) * N) : nullptr;
    const uint2* br = bias ? reinterpret_cast<const uint2*>(bias + static_cast<int64_t>(g) * N) : nullptr;
    float4* yr = reinterpret_cast<float4*>(y + dst * N);
    for (int c = threadIdx.x; c < nchunk; c += kFinThreads) {
      const int4 a = __ldcs(ar + c);
      float4 v = make_float4(__fmul_rn(__int2float_rn(a.x), ts), __fmul_rn(__int2float_rn(a.y), ts),
                             __fmul_rn(__int2float_rn(a.z), ts), __fmul_rn(__int2float_rn(a.w), ts));
      if (wr) {
        const float4 w = wr[c];
        v = make_float4(__fmul_rn(v.x, w.x), __fmul_rn(v.y, w.y), __fmul_rn(v.z, w.z), __fmul_rn(v.w, w.w));
      }
      if (br) {
        const uint2 raw = br[c];
        const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v = make_float4(__fadd_rn(v.x, b0.x), __fadd_rn(v.y, b0.y), __fadd_rn(v.z, b1.x), __fadd_rn(v.w, b1.y));
      }
      v = make_float4(__fmul_rn(v.x, lg), __fmul_rn(v.y, lg), __fmul_rn(v.z, lg), __fmul_rn(v.w, lg));
      atomicAdd(yr + c, v);   // one 16-byte reduction at the L2
    }
  }
}

}  // namespace tab

using namespace tab;

extern "C" int tab_grouped_matmul_finalize_routing_workspace_bytes(int64_t M, int64_t N, size_t* bytes) {
  if (!bytes || M < 0 || N <= 0) return fail(TAB_ERR_BAD_ARG, "grouped_matmul_finalize_routing: M=%lld N=%lld", (long long)M, (long long)N);
  *bytes = (static_cast<size_t>(M) * N * 4 + 255) / 256 * 256;
  return TAB_OK;
}

extern "C" int tab_grouped_matmul_finalize_routing(const int8_t* x, const int8_t* packed_weight, const float* scale,
                                                   const void* bias, const float* per_token_scale,
                                                   const int64_t* group_list, int group_list_type, int64_t M,
                                                   int64_t Kd, int64_t N, int64_t E, const void* shared_input,
                                                   int64_t shared_rows, float shared_input_weight,
                                                   int64_t shared_input_offset, const float* logit,
                                                   const void* row_index, int row_index_dtype, int64_t output_bs,
                                                   float* y, void* workspace, size_t workspace_bytes,
                                                   int64_t expected_rows_per_group, tab_stream_t stream) {
  const char* op = "grouped_matmul_finalize_routing";
  if (M < 0 || N <= 0 || Kd <= 0 || E <= 0 || output_bs < 0 || shared_rows < 0)
    return fail(TAB_ERR_BAD_ARG, "%s: M=%lld Kd=%lld N=%lld E=%lld output_bs=%lld", op, (long long)M, (long long)Kd, (long long)N, (long long)E, (long long)output_bs);
  if (row_index_dtype != TAB_I32 && row_index_dtype != 4 /* int64 */)
    return fail(TAB_ERR_UNSUPPORTED, "%s: row_index dtype %d (want 3 or 4)", op, row_index_dtype);
  if (group_list_type != 0 && group_list_type != 1) return fail(TAB_ERR_BAD_ARG, "%s: group_list_type %d", op, group_list_type);
  if (E > kMaxDsqGroups) return fail(TAB_ERR_UNSUPPORTED, "%s: more than %d groups", op, kMaxDsqGroups);
  if (shared_input && (shared_input_offset < 0 || shared_input_offset + shared_rows > output_bs))
    return fail(TAB_ERR_BAD_ARG, "%s: shared rows [%lld, %lld) outside the %lld output rows", op, (long long)shared_input_offset, (long long)(shared_input_offset + shared_rows), (long long)output_bs);
  if (output_bs == 0) return TAB_OK;
  if (!y) return fail(TAB_ERR_BAD_ARG, "%s: null output", op);
  if (M > 0 && (!row_index || !workspace)) return fail(TAB_ERR_BAD_ARG, "%s: null pointer", op);
  if (N % 4 != 0 || !aligned16(y) || !aligned16(workspace) || (scale && !aligned16(scale)) || (bias && (reinterpret_cast<uintptr_t>(bias) & 7u)) ||
      (shared_input && (reinterpret_cast<uintptr_t>(shared_input) & 7u)))
    return fail(TAB_ERR_ALIGNMENT, "%s: N=%lld must be a multiple of 4 and the pointers 16-byte aligned", op, (long long)N);
  size_t need = 0;
  tab_grouped_matmul_finalize_routing_workspace_bytes(M, N, &need);
  if (M > 0 && workspace_bytes < need) return fail(TAB_ERR_WORKSPACE, "%s: workspace %zu < %zu bytes", op, workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  int32_t* acc = static_cast<int32_t*>(workspace);
  if (M > 0) {
    const int rc = tab_grouped_matmul_w8a8(x, packed_weight, nullptr, nullptr, nullptr, group_list, group_list_type, M, Kd, N, E, TAB_I32, acc,
                                           expected_rows_per_group, stream);
    if (rc != TAB_OK) return rc;
  }
  finalize_init_kernel<<<grid_for(output_bs, 8), kFinThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(shared_input), shared_rows,
                                                                      shared_input_offset, shared_input_weight, output_bs, (int)N, y);
  int rc = check_launch(op);
  if (rc != TAB_OK || M == 0) return rc;
  const size_t smem = static_cast<size_t>(E) * sizeof(int);
  const int grid = grid_for(M, 8);
  const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(bias);
  if (row_index_dtype == TAB_I32)
    finalize_scatter_kernel<int32_t><<<grid, kFinThreads, smem, st>>>(acc, scale, b, per_token_scale, group_list, group_list_type == 0, (int)E, logit,
                                                                     static_cast<const int32_t*>(row_index), M, (int)N, output_bs, y);
  else
    finalize_scatter_kernel<int64_t><<<grid, kFinThreads, smem, st>>>(acc, scale, b, per_token_scale, group_list, group_list_type == 0, (int)E, logit,
                                                                     static_cast<const int64_t*>(row_index), M, (int)N, output_bs, y);
  return check_launch(op);
}
