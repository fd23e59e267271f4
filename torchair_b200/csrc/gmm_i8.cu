// Grouped int8 GEMM for the W8A8 MoE experts on sm_100a (npu_grouped_matmul, and its fusion with
// npu_dequant_swiglu_quant).
//
// Layout.  The weights are the stationary 128-row MMA operand ("A": 128 output channels x K), the tokens of
// one expert the narrow one ("B": NT tokens x K, NT in {16..256}), so a decode batch with a handful of rows
// per expert streams every weight byte exactly once at MMA N = 16 instead of padding tokens to 128 rows.
// Both operands are K-major int8 in 128-byte-swizzled shared memory, written by TMA (no multicast) and read
// by tcgen05.mma.kind::i8 through shared-memory descriptors; the int32 accumulators live in tensor memory:
// lane = output channel, column = token.  A CTA tile is two accumulators: channels [c, c+128) and either
// [c+128, c+256) (plain GEMM) or the matching "up" channels [I+c, I+c+128) (gate_up GEMM with the SwiGLU
// epilogue), so that one thread holds gate and up of the same channel.
//
// Schedule.  Persistent CTAs (one per SM), each walks work items w = blockIdx.x, +gridDim.x, ... of the list
// (expert, channel tile, token tile) that every CTA derives from the device-resident group_list, so no host
// read of the counts is needed.  Warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 =
// epilogue.  Shared-memory stages and (for NT <= 128) two accumulator buffers are handed over with mbarriers.
// Every wait is bounded: on expiry the CTA records a code in g_gmm_status, drains and leaves.
#include <cuda.h>

#include <mutex>

#include <stdlib.h>
#include <string.h>

#include "gmm_common.cuh"
#include "gmm_i8_prefill.cuh"
#include "gmm_i8_pair.cuh"

namespace tab {

template <int NT>
struct GmmCfg {
  static constexpr int kStageBytes = 2 * kWTileBytes + NT * kBlockK;
  static constexpr int kTableBytes = 2 * (kMaxGroups + 1) * 4;
  static constexpr int kCtrlBytes = 256;
  static constexpr int kStagesFit = (kSmemLimit - 1024 - kTableBytes - kCtrlBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kBufs = NT <= 128 ? 2 : 1;
  static constexpr int kTmemCols = kBufs * 2 * NT < 32 ? 32 : kBufs * 2 * NT;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kCtrlBytes + kTableBytes;
};

template <int NT, bool FUSED>
__global__ void __launch_bounds__(kGmmThreads, 1)
gmm_i8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GmmParams p) {
  using Cfg = GmmCfg<NT>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kBufs = Cfg::kBufs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t tiles_addr = ptx::smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
  // barrier indices: full[s] = s, empty[s] = kStages + s, tfull[b] = 2*kStages + b, tempty[b] = 2*kStages + kBufs + b,
  // drain = 2*kStages + 2*kBufs
  const uint32_t bar0 = ptx::smem_u32(bars);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto bar_tfull = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto bar_tempty = [&](int b) { return bar0 + 8u * (2 * kStages + kBufs + b); };
  const uint32_t bar_drain = bar0 + 8u * (2 * kStages + 2 * kBufs);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kStages * Cfg::kStageBytes + 224);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  int* s_start = reinterpret_cast<int*>(smem + kStages * Cfg::kStageBytes + Cfg::kCtrlBytes);  // [E+1] first row
  int* s_pref = s_start + (kMaxGroups + 1);                                                   // [E+1] token tiles before e

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < kBufs; ++b) {
      ptx::mbar_init(bar_tfull(b), 1);
      ptx::mbar_init(bar_tempty(b), 4);
    }
    ptx::mbar_init(bar_drain, 1);
    *s_abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_x);
  }
  if (warp == 1) ptx::tmem_alloc<Cfg::kTmemCols>(ptx::smem_u32(s_tmem));
  if (warp == 0) {
    build_group_tables(p, NT, lane, s_start, s_pref);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = *s_tmem;
  const int total_items = s_pref[E] * p.chan_tiles;
  const int num_kb = (p.Kd + kBlockK - 1) / kBlockK;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long arms = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
        const int ch0 = FUSED ? it.ct * 128 : it.ct * 256;
        const int ch1 = FUSED ? p.half + it.ct * 128 : it.ct * 256 + 128;
        const int row0 = s_start[it.e] + it.tt * NT;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_empty(stage), phase ^ 1u, s_abort, 1, p.wait_cycles)) { ok = false; break; }
          const uint32_t st = tiles_addr + stage * Cfg::kStageBytes;
          ptx::mbar_expect_tx(bar_full(stage), Cfg::kStageBytes);
          ptx::tma_load_3d(st, &tm_w, bar_full(stage), kb * kBlockK, ch0, it.e);
          ptx::tma_load_3d(st + kWTileBytes, &tm_w, bar_full(stage), kb * kBlockK, ch1, it.e);
          ptx::tma_load_2d(st + 2 * kWTileBytes, &tm_x, bar_full(stage), kb * kBlockK, row0);
          ++arms;
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Let the copies already in flight land before the CTA's shared memory goes away.
        for (int s = 0; s < kStages; ++s) {
          const long long a = arms / kStages + (s < arms % kStages ? 1 : 0);
          if (a > 0) {
            const long long t0 = clock64();
            while (!ptx::mbar_try_wait(bar_full(s), static_cast<uint32_t>((a - 1) & 1)) && clock64() - t0 < p.wait_cycles) {}
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_i8(128, NT);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        if (!bounded_wait(bar_tempty(buf), tphase ^ 1u, s_abort, 2, p.wait_cycles)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d0 = tmem_base + buf * 2 * NT;
        const uint32_t d1 = d0 + NT;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_full(stage), phase, s_abort, 3, p.wait_cycles)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t st = tiles_addr + stage * Cfg::kStageBytes;
          const uint64_t a0 = ptx::smem_desc_k128(st);
          const uint64_t a1 = ptx::smem_desc_k128(st + kWTileBytes);
          const uint64_t b = ptx::smem_desc_k128(st + 2 * kWTileBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k) {
            const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
            ptx::mma_i8(d0, a0 + 2 * k, b + 2 * k, idesc, acc);
            ptx::mma_i8(d1, a1 + 2 * k, b + 2 * k, idesc, acc);
          }
          ptx::mma_commit(bar_empty(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit(bar_tfull(buf));
        if (++buf == kBufs) { buf = 0; tphase ^= 1u; }
      }
      if (!ok) {
        // Wait (bounded) for whatever was issued before tensor memory is released.
        ptx::mma_commit(bar_drain);
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(bar_drain, 0) && clock64() - t0 < p.wait_cycles) {}
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 cover TMEM lane quarters 2, 3, 0, 1 ----------------
    const int quarter = warp & 3;
    const int c_local = quarter * 32 + lane;
    int buf = 0;
    uint32_t tphase = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x) {
      int got = 0;
      if (lane == 0) got = bounded_wait(bar_tfull(buf), tphase, s_abort, 4, p.wait_cycles) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      ptx::tc_fence_after();
      const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
      const int row0 = s_start[it.e] + it.tt * NT;
      const int cnt = s_start[it.e + 1] - s_start[it.e];
      const int nvalid = min(NT, cnt - it.tt * NT);
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * 2 * NT;
      if constexpr (FUSED) {
        const int cg = it.ct * 128 + c_local;
        const bool cvalid = cg < p.half;
        const float wg = (cvalid && p.w_scale) ? p.w_scale[static_cast<int64_t>(it.e) * p.N + cg] : 1.f;
        const float wu = (cvalid && p.w_scale) ? p.w_scale[static_cast<int64_t>(it.e) * p.N + p.half + cg] : 1.f;
        for (int col0 = 0; col0 < nvalid; col0 += 16) {
          int g[16], u[16];
          __syncwarp();
          ptx::tmem_ld16(t0 + col0, g);
          ptx::tmem_ld16(t0 + NT + col0, u);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int row = row0 + col0 + j;
            const bool rvalid = col0 + j < nvalid;   // uniform over the warp
            float h = 0.f;
            if (rvalid) {
              const float ts = p.tok_scale ? p.tok_scale[row] : 1.f;
              const float gv = __fmul_rn(__fmul_rn(__int2float_rn(g[j]), ts), wg);
              const float uv = __fmul_rn(__fmul_rn(__int2float_rn(u[j]), ts), wu);
              h = silu_mul(p.activate_left ? gv : uv, p.activate_left ? uv : gv);   // one SwiGLU, operands picked first
              if (cvalid) p.h_out[static_cast<int64_t>(row) * p.half + cg] = h;
              const float m = warp_max(cvalid ? fabsf(h) : 0.f);
              if (lane == 0) atomicMax(p.amax + row, __float_as_uint(m));
            }
          }
        }
      } else {
        const int c0 = it.ct * 256 + c_local;
        const int c1 = c0 + 128;
        const bool v0 = c0 < p.N, v1 = c1 < p.N;
        const float w0 = (v0 && p.w_scale) ? p.w_scale[static_cast<int64_t>(it.e) * p.N + c0] : 1.f;
        const float w1 = (v1 && p.w_scale) ? p.w_scale[static_cast<int64_t>(it.e) * p.N + c1] : 1.f;
        const int bias0 = (v0 && p.bias) ? p.bias[static_cast<int64_t>(it.e) * p.N + c0] : 0;
        const int bias1 = (v1 && p.bias) ? p.bias[static_cast<int64_t>(it.e) * p.N + c1] : 0;
        for (int col0 = 0; col0 < nvalid; col0 += 16) {
          int a[16], b[16];
          __syncwarp();
          ptx::tmem_ld16(t0 + col0, a);
          ptx::tmem_ld16(t0 + NT + col0, b);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            a[j] += bias0;
            b[j] += bias1;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (col0 + j < nvalid) {
              const int64_t row = row0 + col0 + j;
              if (p.out_dtype == TAB_I32) {
                int* o = static_cast<int*>(p.out) + row * p.N;
                if (v0) o[c0] = a[j];
                if (v1) o[c1] = b[j];
              } else {
                const float ts = p.tok_scale ? p.tok_scale[row] : 1.f;
                const float f0 = __fmul_rn(__fmul_rn(__int2float_rn(a[j]), ts), w0);
                const float f1 = __fmul_rn(__fmul_rn(__int2float_rn(b[j]), ts), w1);
                uint8_t* orow = out_row_ptr(p, row, 2);
                if (orow == nullptr) continue;             // address table says: no destination for this row
                if (p.out_dtype == TAB_BF16) {
                  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(orow);
                  if (v0) o[c0] = __float2bfloat16_rn(f0);
                  if (v1) o[c1] = __float2bfloat16_rn(f1);
                } else {
                  __half* o = reinterpret_cast<__half*>(orow);
                  if (v0) o[c0] = __float2half_rn(f0);
                  if (v1) o[c1] = __float2half_rn(f1);
                }
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));
      if (++buf == kBufs) { buf = 0; tphase ^= 1u; }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<Cfg::kTmemCols>(tmem_base);
  }
}

// packed[e, n, k] = weight[e, k, n]; 64x64-byte tiles through shared memory.
__global__ void __launch_bounds__(256) prepack_kernel(const int8_t* __restrict__ w, int Kd, int N, int8_t* __restrict__ out) {
  __shared__ int8_t tile[64][64 + 4];
  const int64_t e = blockIdx.z;
  const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int8_t* src = w + e * static_cast<int64_t>(Kd) * N;
  int8_t* dst = out + e * static_cast<int64_t>(Kd) * N;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int kk = i >> 6, nn = i & 63;
    tile[kk][nn] = (k0 + kk < Kd && n0 + nn < N) ? src[static_cast<int64_t>(k0 + kk) * N + n0 + nn] : int8_t(0);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int nn = i >> 6, kk = i & 63;
    if (n0 + nn < N && k0 + kk < Kd) dst[static_cast<int64_t>(n0 + nn) * Kd + k0 + kk] = tile[kk][nn];
  }
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

static int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kNumSMs;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMs;
    cached[dev] = n;
  }
  return cached[dev];
}

// Weight map: 3-D (K, channel, expert), box 128 bytes x 128 channels; token map: 2-D (K, row), box 128 x NT.
static int make_maps(const int8_t* x, const int8_t* wp, int64_t M, int64_t Kd, int64_t N, int64_t E, int nt,
                     CUtensorMap* tm_w, CUtensorMap* tm_x, CUtensorMap* tm_w64 = nullptr) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(TAB_ERR_CUDA, "grouped_matmul: cuTensorMapEncodeTiled is not available from the driver");
  for (int half_box = 0; half_box < (tm_w64 ? 2 : 1); ++half_box) {      // 128-channel boxes; 64-channel boxes for the pair kernel's gate | up halves
    cuuint64_t dims[3] = {(cuuint64_t)Kd, (cuuint64_t)N, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)Kd, (cuuint64_t)(Kd * N)};
    cuuint32_t box[3] = {kBlockK, half_box ? 64u : 128u, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = enc(half_box ? tm_w64 : tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(wp), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAB_ERR_CUDA, "grouped_matmul: weight tensor map rejected (CUresult %d)", (int)r);
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)Kd, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)Kd};
    cuuint32_t box[2] = {kBlockK, (cuuint32_t)nt};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(x), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TAB_ERR_CUDA, "grouped_matmul: activation tensor map rejected (CUresult %d)", (int)r);
  }
  return TAB_OK;
}

// Tuning and safety knobs from the environment, read once when the library is first used:
//   TAB_GMM_NT=16|32|64|128|256          token-tile width of the decode orientation (default: from M / E)
//   TAB_GMM_ORIENTATION=decode|prefill|pair   kernel (default: by the expected rows per group, see use_prefill / use_pair)
//   TAB_GMM_WAIT_MS=<ms>                 bound of every device-side wait inside the GEMM kernels (default 2000)
struct GmmEnv {
  int nt = 0;
  int orientation = 0;   // 0 auto, 1 decode, 2 prefill (one CTA per tile), 3 prefill on CTA pairs
  long long wait_cycles = 2000 * kCyclesPerMs;
  GmmEnv() {
    if (const char* f = getenv("TAB_GMM_NT")) {
      const int v = atoi(f);
      if (v == 16 || v == 32 || v == 64 || v == 128 || v == 256) nt = v;
    }
    if (const char* f = getenv("TAB_GMM_ORIENTATION")) {
      if (strcmp(f, "decode") == 0) orientation = 1;
      if (strcmp(f, "prefill") == 0) orientation = 2;
      if (strcmp(f, "pair") == 0) orientation = 3;
    }
    if (const char* f = getenv("TAB_GMM_WAIT_MS")) {
      const long long ms = atoll(f);
      if (ms >= 1 && ms <= 600000) wait_cycles = ms * kCyclesPerMs;
    }
  }
};
static const GmmEnv& gmm_env() {
  static const GmmEnv env;
  return env;
}

// Rows per group the tiling is chosen for: the caller's expectation when it gave one (the first element of the
// operator's tuning_config), else the allocated rows spread evenly.  With expert parallelism x is sized for the worst
// case (every rank sending everything here), so M / E can be many times the rows that actually arrive.
static double rows_per_group(int64_t M, int64_t E, int64_t expected) {
  return expected > 0 ? static_cast<double>(expected) : static_cast<double>(M) / static_cast<double>(E);
}

// Token-tile width of the decode orientation: the smallest of 16..256 that holds 1.5 x the average rows per expert.
static int pick_nt(double avg) {
  if (gmm_env().nt != 0) return gmm_env().nt;
  const int opts[5] = {16, 32, 64, 128, 256};
  for (int i = 0; i < 5; ++i)
    if (opts[i] >= 1.5 * avg) return opts[i];
  return 256;
}

template <int NT, bool FUSED>
static int launch_one(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GmmParams& p, int grid, cudaStream_t st) {
  using Cfg = GmmCfg<NT>;
  static_assert(Cfg::kStages >= 2, "at least two shared-memory stages");
  static_assert(2 * Cfg::kStages * 8 + 2 * Cfg::kBufs * 8 + 8 <= 224, "barriers overflow the control block");
  cudaError_t e = cudaFuncSetAttribute(gmm_i8_kernel<NT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "grouped_matmul: shared memory opt-in failed: %s", cudaGetErrorString(e));
  gmm_i8_kernel<NT, FUSED><<<grid, kGmmThreads, Cfg::kSmemBytes, st>>>(tm_w, tm_x, p);
  return check_launch("grouped_matmul");
}

// Orientation: experts with many rows run the prefill kernel (128-token tiles, overlapped epilogue); a handful of
// rows per expert run the decode kernel (weights stationary, narrow token tile).
static bool use_prefill(double avg) {
  if (gmm_env().orientation != 0) return gmm_env().orientation >= 2;
  return avg > 64.0;
}

// The CTA-pair kernel computes 256-token tiles: an expert's last tile of 65..255 rows costs a whole tile, and per tile the
// pair's epilogue is as long as that of two one-CTA tiles while its main loop saves operand traffic in proportion to K.
// Measured cross-over (rows per group, counts spread by a quarter around the mean): about 450 rows at K = 7168, 750 at
// K = 4096, 1000 at K = 1536..2048.
static bool use_pair(double avg, int64_t Kd) {
  if (gmm_env().orientation != 0) return gmm_env().orientation == 3;
  if (Kd >= 6144) return avg >= 448.0;
  if (Kd >= 3072) return avg >= 768.0;
  return avg >= 1024.0;
}

template <bool FUSED>
static int launch_prefill(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GmmParams& p, cudaStream_t st) {
  const int64_t max_items = ((static_cast<int64_t>(p.M) + kPfTokens - 1) / kPfTokens + p.E) * p.chan_tiles;
  const int sms = num_sms();
  const int grid = static_cast<int>(max_items < sms ? max_items : sms);
  cudaError_t e = cudaFuncSetAttribute(gmm_i8_prefill_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmemBytes);
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "grouped_matmul: shared memory opt-in failed: %s", cudaGetErrorString(e));
  gmm_i8_prefill_kernel<FUSED><<<grid, kPfThreads, kPfSmemBytes, st>>>(tm_w, tm_x, p);
  return check_launch("grouped_matmul (prefill)");
}

template <bool FUSED>
static int launch_pair(const CUtensorMap& tm_w, const CUtensorMap& tm_w64, const CUtensorMap& tm_x, const GmmParams& p, cudaStream_t st) {
  const int64_t max_items = ((static_cast<int64_t>(p.M) + kPairTokens - 1) / kPairTokens + p.E) * p.chan_tiles;
  const int pairs = num_sms() / 2;
  const int grid = 2 * static_cast<int>(max_items < pairs ? max_items : pairs);
  cudaError_t e = cudaFuncSetAttribute(gmm_i8_pair_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "grouped_matmul: shared memory opt-in failed: %s", cudaGetErrorString(e));
  gmm_i8_pair_kernel<FUSED><<<grid, kPfThreads, kPairSmemBytes, st>>>(tm_w, tm_w64, tm_x, p);
  return check_launch("grouped_matmul (CTA pairs)");
}

template <bool FUSED>
static int launch_gmm(int nt, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GmmParams& p, cudaStream_t st) {
  if (nt == 0) return launch_prefill<FUSED>(tm_w, tm_x, p, st);
  const int64_t max_items = ((static_cast<int64_t>(p.M) + nt - 1) / nt + p.E) * p.chan_tiles;
  const int sms = num_sms();
  const int grid = static_cast<int>(max_items < sms ? max_items : sms);
  switch (nt) {
    case 16: return launch_one<16, FUSED>(tm_w, tm_x, p, grid, st);
    case 32: return launch_one<32, FUSED>(tm_w, tm_x, p, grid, st);
    case 64: return launch_one<64, FUSED>(tm_w, tm_x, p, grid, st);
    case 128: return launch_one<128, FUSED>(tm_w, tm_x, p, grid, st);
    default: return launch_one<256, FUSED>(tm_w, tm_x, p, grid, st);
  }
}

static int check_common(const char* op, const int8_t* x, const int8_t* wp, const int64_t* group_list, int group_list_type,
                        int64_t M, int64_t Kd, int64_t N, int64_t E) {
  if (M < 0 || Kd <= 0 || N <= 0 || E <= 0) return fail(TAB_ERR_BAD_ARG, "%s: M=%lld Kd=%lld N=%lld E=%lld", op, (long long)M, (long long)Kd, (long long)N, (long long)E);
  if (E > kMaxGroups) return fail(TAB_ERR_UNSUPPORTED, "%s: %lld groups (at most %d)", op, (long long)E, kMaxGroups);
  if (M > (1LL << 30) || N > (1LL << 24) || Kd > (1LL << 24)) return fail(TAB_ERR_UNSUPPORTED, "%s: dimension too large", op);
  if (group_list_type != 0 && group_list_type != 1) return fail(TAB_ERR_BAD_ARG, "%s: group_list_type %d", op, group_list_type);
  if (M > 0 && (!x || !wp || !group_list)) return fail(TAB_ERR_BAD_ARG, "%s: null pointer", op);
  if (Kd % 16 != 0) return fail(TAB_ERR_ALIGNMENT, "%s: Kd=%lld must be a multiple of 16", op, (long long)Kd);
  if (!aligned16(x) || !aligned16(wp)) return fail(TAB_ERR_ALIGNMENT, "%s: x and weight must be 16-byte aligned", op);
  return TAB_OK;
}

int launch_quant_from_f32(const float* h, const uint32_t* amax_bits, const int64_t* group_list, int group_list_type,
                          int num_groups, int64_t rows, int cols, int8_t* y, float* scale, cudaStream_t st);

}  // namespace tab

using namespace tab;

extern "C" int tab_prepack_weight_i8(const int8_t* weight, int64_t E, int64_t Kd, int64_t N, int8_t* packed,
                                     tab_stream_t stream) {
  if (!weight || !packed || E <= 0 || Kd <= 0 || N <= 0 || E > 65535) return fail(TAB_ERR_BAD_ARG, "prepack_weight: bad argument");
  if (weight == packed) return fail(TAB_ERR_BAD_ARG, "prepack_weight: in-place relayout is not supported");
  dim3 grid((unsigned)((N + 63) / 64), (unsigned)((Kd + 63) / 64), (unsigned)E);
  if (grid.y > 65535) return fail(TAB_ERR_UNSUPPORTED, "prepack_weight: Kd too large");
  prepack_kernel<<<grid, 256, 0, as_stream(stream)>>>(weight, (int)Kd, (int)N, packed);
  return check_launch("prepack_weight");
}

static int grouped_matmul_plain(const int8_t* x, const int8_t* packed_weight, const float* scale, const float* per_token_scale,
                                const int32_t* bias,
                                const int64_t* group_list, int group_list_type, int64_t M, int64_t Kd, int64_t N, int64_t E,
                                int out_dtype, void* y, const uint64_t* row_dst, int64_t expected_rows_per_group,
                                tab_stream_t stream) {
  int rc = check_common("grouped_matmul", x, packed_weight, group_list, group_list_type, M, Kd, N, E);
  if (rc != TAB_OK) return rc;
  if (out_dtype != TAB_I32 && out_dtype != TAB_BF16 && out_dtype != TAB_F16)
    return fail(TAB_ERR_UNSUPPORTED, "grouped_matmul: output dtype %d (want 3, 5 or 15)", out_dtype);
  if (row_dst && out_dtype == TAB_I32) return fail(TAB_ERR_UNSUPPORTED, "grouped_matmul: a row address table needs a 16-bit output dtype");
  if (M == 0) return TAB_OK;
  if (!y && !row_dst) return fail(TAB_ERR_BAD_ARG, "grouped_matmul: null output");
  const double avg = rows_per_group(M, E, expected_rows_per_group);
  const int nt = use_prefill(avg) ? 0 : pick_nt(avg);     // 0 selects the prefill orientation
  const bool pair = nt == 0 && use_pair(avg, Kd);
  CUtensorMap tm_w, tm_x, tm_w64;
  rc = make_maps(x, packed_weight, M, Kd, N, E, nt == 0 ? kPfTokens : nt, &tm_w, &tm_x, pair ? &tm_w64 : nullptr);
  if (rc != TAB_OK) return rc;
  GmmParams p = {};
  p.group_list = group_list;
  p.group_list_type = group_list_type;
  p.E = (int)E; p.M = (int)M; p.N = (int)N; p.Kd = (int)Kd;
  p.chan_tiles = (int)((N + 255) / 256);
  p.half = 0;
  p.w_scale = out_dtype == TAB_I32 ? nullptr : scale;
  p.tok_scale = out_dtype == TAB_I32 ? nullptr : per_token_scale;
  p.bias = bias;
  p.out = y;
  p.out_dtype = out_dtype;
  p.row_dst = reinterpret_cast<const unsigned long long*>(row_dst);
  p.wait_cycles = gmm_env().wait_cycles;
  if (pair) return launch_pair<false>(tm_w, tm_w64, tm_x, p, as_stream(stream));
  return launch_gmm<false>(nt, tm_w, tm_x, p, as_stream(stream));
}

extern "C" int tab_grouped_matmul_w8a8(const int8_t* x, const int8_t* packed_weight, const float* scale,
                                       const float* per_token_scale, const int32_t* bias, const int64_t* group_list,
                                       int group_list_type, int64_t M, int64_t Kd, int64_t N, int64_t E, int out_dtype, void* y,
                                       int64_t expected_rows_per_group, tab_stream_t stream) {
  return grouped_matmul_plain(x, packed_weight, scale, per_token_scale, bias, group_list, group_list_type, M, Kd, N, E, out_dtype, y,
                              nullptr, expected_rows_per_group, stream);
}

extern "C" int tab_grouped_matmul_w8a8_scatter(const int8_t* x, const int8_t* packed_weight, const float* scale,
                                               const float* per_token_scale, const int64_t* group_list, int group_list_type,
                                               int64_t M, int64_t Kd, int64_t N, int64_t E, int out_dtype,
                                               const uint64_t* row_dst, int64_t expected_rows_per_group,
                                               tab_stream_t stream) {
  if (!row_dst && M > 0) return fail(TAB_ERR_BAD_ARG, "grouped_matmul_scatter: null row address table");
  if ((N * 2) % 16 != 0) return fail(TAB_ERR_ALIGNMENT, "grouped_matmul_scatter: N=%lld must be a multiple of 8", (long long)N);
  return grouped_matmul_plain(x, packed_weight, scale, per_token_scale, nullptr, group_list, group_list_type, M, Kd, N, E, out_dtype,
                              nullptr, row_dst, expected_rows_per_group, stream);
}

extern "C" int tab_grouped_matmul_swiglu_quant_workspace_bytes(int64_t M, int64_t I, size_t* bytes) {
  if (!bytes || M < 0 || I <= 0) return fail(TAB_ERR_BAD_ARG, "grouped_matmul_swiglu_quant: M=%lld I=%lld", (long long)M, (long long)I);
  const size_t amax = (static_cast<size_t>(M) * 4 + 255) / 256 * 256;
  *bytes = amax + static_cast<size_t>(M) * I * 4;
  return TAB_OK;
}

extern "C" int tab_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* packed_weight, const float* weight_scale,
                                               const float* x_scale, const int64_t* group_list, int group_list_type,
                                               int64_t M, int64_t Kd, int64_t I, int64_t E, int activate_left,
                                               int8_t* yq, float* y_scale, void* workspace, size_t workspace_bytes,
                                               int64_t expected_rows_per_group, tab_stream_t stream) {
  int rc = check_common("grouped_matmul_swiglu_quant", x, packed_weight, group_list, group_list_type, M, Kd, 2 * I, E);
  if (rc != TAB_OK) return rc;
  if (M == 0) return TAB_OK;
  if (!yq || !y_scale || !workspace) return fail(TAB_ERR_BAD_ARG, "grouped_matmul_swiglu_quant: null pointer");
  if (I % 8 != 0 || !aligned16(yq) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(TAB_ERR_ALIGNMENT, "grouped_matmul_swiglu_quant: I=%lld must be a multiple of 8, yq 16-byte and workspace 256-byte aligned", (long long)I);
  size_t need = 0;
  tab_grouped_matmul_swiglu_quant_workspace_bytes(M, I, &need);
  if (workspace_bytes < need) return fail(TAB_ERR_WORKSPACE, "grouped_matmul_swiglu_quant: workspace %zu < %zu bytes", workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  const size_t amax_bytes = (static_cast<size_t>(M) * 4 + 255) / 256 * 256;
  unsigned int* amax = static_cast<unsigned int*>(workspace);
  float* h = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + amax_bytes);
  cudaError_t ce = cudaMemsetAsync(amax, 0, amax_bytes, st);
  if (ce != cudaSuccess) return fail(TAB_ERR_CUDA, "grouped_matmul_swiglu_quant: memset: %s", cudaGetErrorString(ce));
  const double avg = rows_per_group(M, E, expected_rows_per_group);
  const int nt = use_prefill(avg) ? 0 : pick_nt(avg);     // 0 selects the prefill orientation
  const bool pair = nt == 0 && use_pair(avg, Kd);
  CUtensorMap tm_w, tm_x, tm_w64;
  rc = make_maps(x, packed_weight, M, Kd, 2 * I, E, nt == 0 ? kPfTokens : nt, &tm_w, &tm_x, pair ? &tm_w64 : nullptr);
  if (rc != TAB_OK) return rc;
  GmmParams p = {};
  p.group_list = group_list;
  p.group_list_type = group_list_type;
  p.E = (int)E; p.M = (int)M; p.N = (int)(2 * I); p.Kd = (int)Kd;
  p.chan_tiles = (int)((I + 127) / 128);
  p.half = (int)I;
  p.w_scale = weight_scale;
  p.tok_scale = x_scale;
  p.h_out = h;
  p.amax = amax;
  p.activate_left = activate_left;
  p.wait_cycles = gmm_env().wait_cycles;
  rc = pair ? launch_pair<true>(tm_w, tm_w64, tm_x, p, st) : launch_gmm<true>(nt, tm_w, tm_x, p, st);
  if (rc != TAB_OK) return rc;
  return launch_quant_from_f32(h, amax, group_list, group_list_type, (int)E, M, (int)I, yq, y_scale, st);
}

extern "C" int tab_gmm_status_reset(tab_stream_t stream) {
  cudaError_t e = cudaStreamSynchronize(as_stream(stream));
  const int zero = 0;
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_gmm_status, &zero, sizeof(int));
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "gmm_status_reset: %s", cudaGetErrorString(e));
  return TAB_OK;
}

extern "C" int tab_gmm_status(int* status_host, tab_stream_t stream) {
  if (!status_host) return fail(TAB_ERR_BAD_ARG, "gmm_status: null pointer");
  cudaError_t e = cudaStreamSynchronize(as_stream(stream));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(status_host, g_gmm_status, sizeof(int));
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "gmm_status: %s", cudaGetErrorString(e));
  if (*status_host != 0) return fail(TAB_ERR_TIMEOUT, "grouped_matmul: device-side wait %d gave up", *status_host);
  return TAB_OK;
}
