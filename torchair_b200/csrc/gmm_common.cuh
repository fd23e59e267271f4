// Pieces shared by the two grouped-GEMM kernels (decode orientation in gmm_i8.cu, prefill orientation in
// gmm_i8_prefill.cuh): launch parameters, the bounded mbarrier wait, and the work-item list derived from group_list.
#pragma once

#include <cuda.h>

#include "ptx_sm100.cuh"
#include "tab_common.cuh"

namespace tab {

// Status word of the grouped GEMMs on this device: 0, or the code of the bounded wait that gave up (tab_gmm_status).
// This header is included by exactly one translation unit (gmm_i8.cu).
__device__ int g_gmm_status = 0;

constexpr int kGmmThreads = 192;
constexpr int kBlockK = 128;               // bytes of K per stage row = one swizzle span
constexpr int kWTileBytes = 128 * kBlockK;  // one 128-channel weight tile
constexpr int kMaxGroups = 1024;
constexpr long long kCyclesPerMs = 2000000LL;   // SM clock ticks per millisecond at the top clock (1965 MHz), rounded up
constexpr int kSmemLimit = 232448;

struct GmmParams {
  const int64_t* group_list;
  int group_list_type;
  int E;
  int M;
  int N;           // channels of the packed weight (plain: N; fused: 2*I)
  int Kd;
  int chan_tiles;  // plain: ceil(N/256); fused: ceil(I/128)
  int half;        // fused: I
  const float* w_scale;    // [E, N] or null
  const int32_t* bias;     // plain: [E, N] added to the int32 accumulators before anything else, or null
  const float* tok_scale;  // [M] or null
  void* out;               // plain: [M, N] of out_dtype
  int out_dtype;
  const unsigned long long* row_dst;   // plain, 16-bit output: address of every output row (may be peer memory), or null
  float* h_out;            // fused: [M, I] fp32
  unsigned int* amax;      // fused: [M] row amax as fp32 bits
  int activate_left;
  long long wait_cycles;   // bound of every device-side wait, in SM clock ticks (TAB_GMM_WAIT_MS, default 2000 ms)
};

// Waits for a phase of an mbarrier; gives up after `limit` clock ticks or when another role already gave up.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                             long long limit) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = code;
        atomicCAS(&g_gmm_status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// First byte of output row `row`: the row's own address when a table is given (0 there = the row belongs to no
// destination and must not be stored), else row-major in p.out.  Callers skip the row on a null result.
__device__ __forceinline__ uint8_t* out_row_ptr(const GmmParams& p, int64_t row, int esz) {
  return p.row_dst ? reinterpret_cast<uint8_t*>(p.row_dst[row]) : static_cast<uint8_t*>(p.out) + row * p.N * esz;
}

struct WorkItem {
  int e, ct, tt;
};

__device__ __forceinline__ WorkItem decode_item(int w, int chan_tiles, int E, const int* s_pref) {
  const int q = w / chan_tiles;
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_pref[mid] <= q) lo = mid; else hi = mid;
  }
  const int ntt = s_pref[lo + 1] - s_pref[lo];
  const int local = w - chan_tiles * s_pref[lo];
  WorkItem it;
  it.e = lo;
  it.ct = local / ntt;
  it.tt = local - it.ct * ntt;
  return it;
}


// Row range [s_start[e], s_start[e+1]) and number of token tiles before expert e (s_pref), computed by one warp
// from the device-resident group_list; tile = rows per token tile.  Arrays hold E + 1 entries.
__device__ __forceinline__ void build_group_tables(const GmmParams& p, int tile, int lane, int* s_start, int* s_pref) {
  const int E = p.E;
  long long run_rows = 0;
  int run_tiles = 0;
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    long long c = 0;
    if (e < E) {
      const long long g = p.group_list[e];
      c = p.group_list_type == 1 ? g : g - (e > 0 ? p.group_list[e - 1] : 0);
      if (c < 0) c = 0;
    }
    long long incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    long long end = run_rows + incl, start = end - c;
    if (end > p.M) end = p.M;
    if (start > p.M) start = p.M;
    const int cnt = static_cast<int>(end - start);
    const int tiles = (cnt + tile - 1) / tile;
    int tincl = tiles;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, tincl, o);
      if (lane >= o) tincl += t;
    }
    if (e < E) {
      s_start[e] = static_cast<int>(start);
      s_pref[e] = run_tiles + tincl - tiles;
    }
    run_rows += __shfl_sync(0xffffffffu, incl, 31);
    run_tiles += __shfl_sync(0xffffffffu, tincl, 31);
  }
  if (lane == 0) {
    s_start[E] = static_cast<int>(run_rows > p.M ? p.M : run_rows);
    s_pref[E] = run_tiles;
  }
}

}  // namespace tab
