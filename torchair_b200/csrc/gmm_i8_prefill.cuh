// Grouped int8 GEMM, prefill orientation: tokens are the 128-row MMA operand, weight channels the 256-wide one.
//
// When experts own hundreds of rows the GEMM is tensor-bound and the epilogue has to hide behind the main loop.
// Here a CTA tile is 128 tokens x 256 channel columns in ONE accumulator (lane = token, column = channel), so
//   - two accumulator buffers fit in tensor memory (2 x 256 columns) and the epilogue of tile i overlaps the
//     MMAs of tile i+1;
//   - a thread owns one token row: its activation scale is a register, the row amax of the fused SwiGLU epilogue
//     accumulates in a register (one atomicMax per thread and tile), and stores are 16-byte vectors along the row;
//   - for the gate_up GEMM the 256 columns are [128 gate channels | the matching 128 up channels] (two TMA boxes
//     into one operand tile), so gate and up of a channel meet in the same thread.
// Roles, barriers, bounded waits and the work-item list are those of the decode-orientation kernel.
//
// Narrow tiles: an expert's last token tile often holds only a few rows (256 +- 16 rows per expert leave a third tile
// of a dozen rows), and as a 128-row operand it would cost a full tile of MMA work.  A tile with at most kPfNarrowMax
// valid rows is therefore computed with the operands swapped, out of the very same shared-memory stage: each
// 128-channel half of the weight tile is the 128-row operand, the token tile the N operand with N = rows rounded up
// to 16, into two accumulators (columns 0.. and 128.. of the buffer; lane = channel, column = token).  MMA work
// shrinks in proportion to the rows; the epilogue for such tiles runs per channel lane and is masked per token.
#pragma once

#include "gmm_common.cuh"

namespace tab {

constexpr int kPfTokens = 128;                       // token rows per tile (MMA M)
constexpr int kPfCols = 256;                         // channel columns per tile (MMA N)
constexpr int kPfATile = kPfTokens * kBlockK;        // 16 KB
constexpr int kPfBTile = kPfCols * kBlockK;          // 32 KB
constexpr int kPfStageBytes = kPfATile + kPfBTile;   // 48 KB
constexpr int kPfStages = 4;
constexpr int kPfBufs = 2;
constexpr int kPfCtrlBytes = 256;
constexpr int kPfScaleBytes = 2 * kPfCols * 4;       // weight scales of the tile, double-buffered
constexpr int kPfTableBytes = (2 * (kMaxGroups + 1) * 4 + 15) / 16 * 16;
constexpr int kPfOutPitch = 80;                      // bytes per staged row: 32 16-bit values + 16 bytes of padding
constexpr int kPfOutStageBytes = 8 * 32 * kPfOutPitch;   // per epilogue warp: 32 rows x 32 columns of 16-bit output
constexpr int kPfSmemBytes = 1024 + kPfStages * kPfStageBytes + kPfCtrlBytes + kPfScaleBytes + kPfTableBytes + kPfOutStageBytes;
static_assert(kPfSmemBytes <= kSmemLimit, "prefill GEMM shared memory");

constexpr int kPfNarrowMax = 64;                     // token tiles with at most this many valid rows swap the operands
constexpr int kPfEpiWarps = 8;                       // two warps per TMEM lane quarter, each takes half of the columns
constexpr int kPfThreads = 64 + kPfEpiWarps * 32;    // producer warp + MMA warp + epilogue warps

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Epilogue of a narrow tile (operands swapped): this thread's TMEM lane is channel `c_l` of the tile's 128-channel
// halves, columns are tokens.  Plain GEMM: accumulator 0 holds channels [0,128) of the tile, accumulator 1 (128 columns
// further) channels [128,256); the two warps of a lane quarter take one accumulator each.  Fused gate_up: accumulator 0
// holds gate, accumulator 1 the matching up channels; the two warps alternate over the 16-token column chunks.  The
// arithmetic per element is that of the wide tiles, so results do not depend on which form a tile took.
template <bool FUSED>
__device__ __forceinline__ void pf_narrow_epilogue(const GmmParams& p, const WorkItem& it, const float* ws, uint32_t t0,
                                                   int row0, int nvalid, int c_l, int lane, int chalf) {
  const int nv16 = (nvalid + 15) & ~15;
  if constexpr (FUSED) {
    const int ch = it.ct * 128 + c_l;                 // channel inside the half
    const bool cvalid = ch < p.half;
    const float wg = ws[c_l], wu = ws[128 + c_l];
#pragma unroll 1
    for (int c = chalf * 16; c < nv16; c += 32) {
      int g[16], u[16];
      __syncwarp();
      ptx::tmem_ld16(t0 + c, g);
      ptx::tmem_ld16(t0 + 128 + c, u);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const bool tvalid = c + j < nvalid;           // uniform over the warp
        const int row = row0 + c + j;
        const float ts = (tvalid && p.tok_scale) ? p.tok_scale[row] : 1.f;
        const float gv = __fmul_rn(__fmul_rn(__int2float_rn(g[j]), ts), wg);
        const float uv = __fmul_rn(__fmul_rn(__int2float_rn(u[j]), ts), wu);
        const float h = silu_mul(p.activate_left ? gv : uv, p.activate_left ? uv : gv);
        if (tvalid) {
          if (cvalid) __stcs(p.h_out + static_cast<int64_t>(row) * p.half + ch, h);
          const float m = warp_max(cvalid ? fabsf(h) : 0.f);
          if (lane == 0) atomicMax(p.amax + row, __float_as_uint(m));
        }
      }
    }
  } else {
    const int ch = it.ct * 256 + chalf * 128 + c_l;
    const bool cvalid = ch < p.N;
    const float wv = ws[chalf * 128 + c_l];
    const int bias = (cvalid && p.bias) ? p.bias[static_cast<int64_t>(it.e) * p.N + ch] : 0;
#pragma unroll 1
    for (int c = 0; c < nv16; c += 16) {
      int a[16];
      __syncwarp();
      ptx::tmem_ld16(t0 + chalf * 128 + c, a);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        a[j] += bias;
        const int row = row0 + c + j;
        if (c + j < nvalid && cvalid) {
          if (p.out_dtype == TAB_I32) {
            static_cast<int*>(p.out)[static_cast<int64_t>(row) * p.N + ch] = a[j];
          } else {
            const float ts = p.tok_scale ? p.tok_scale[row] : 1.f;
            const float f = __fmul_rn(__fmul_rn(__int2float_rn(a[j]), ts), wv);
            uint8_t* orow = out_row_ptr(p, row, 2);
            if (orow == nullptr) continue;               // address table says: no destination for this row
            if (p.out_dtype == TAB_BF16) reinterpret_cast<__nv_bfloat16*>(orow)[ch] = __float2bfloat16_rn(f);
            else reinterpret_cast<__half*>(orow)[ch] = __float2half_rn(f);
          }
        }
      }
    }
  }
}

template <bool FUSED>
__global__ void __launch_bounds__(kPfThreads, 1)
gmm_i8_prefill_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t tiles_addr = ptx::smem_u32(smem);
  uint8_t* ctrl = smem + kPfStages * kPfStageBytes;
  const uint32_t bar0 = ptx::smem_u32(ctrl);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kPfStages + s); };
  auto bar_tfull = [&](int b) { return bar0 + 8u * (2 * kPfStages + b); };
  auto bar_tempty = [&](int b) { return bar0 + 8u * (2 * kPfStages + kPfBufs + b); };
  const uint32_t bar_drain = bar0 + 8u * (2 * kPfStages + 2 * kPfBufs);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(ctrl + 224);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_got = reinterpret_cast<volatile int*>(s_tmem + 2);   // [2] outcome of the epilogue's wait, per buffer
  float* s_wscale = reinterpret_cast<float*>(ctrl + kPfCtrlBytes);     // [2][256]
  int* s_start = reinterpret_cast<int*>(ctrl + kPfCtrlBytes + kPfScaleBytes);
  int* s_pref = s_start + (kMaxGroups + 1);
  uint8_t* s_out = ctrl + kPfCtrlBytes + kPfScaleBytes + kPfTableBytes;   // 16-byte aligned: every part above is

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPfStages; ++s) {
      ptx::mbar_init(bar_full(s), 1);
      ptx::mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < kPfBufs; ++b) {
      ptx::mbar_init(bar_tfull(b), 1);
      ptx::mbar_init(bar_tempty(b), kPfEpiWarps);
    }
    ptx::mbar_init(bar_drain, 1);
    *s_abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_x);
  }
  if (warp == 1) ptx::tmem_alloc<kPfBufs * kPfCols>(ptx::smem_u32(s_tmem));
  if (warp == 0) build_group_tables(p, kPfTokens, lane, s_start, s_pref);
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
        const int ch0 = FUSED ? it.ct * 128 : it.ct * 256;                   // first 128 columns
        const int ch1 = FUSED ? p.half + it.ct * 128 : it.ct * 256 + 128;    // second 128 columns
        const int row0 = s_start[it.e] + it.tt * kPfTokens;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_empty(stage), phase ^ 1u, s_abort, 11, p.wait_cycles)) { ok = false; break; }
          const uint32_t st = tiles_addr + stage * kPfStageBytes;
          ptx::mbar_expect_tx(bar_full(stage), kPfStageBytes);
          ptx::tma_load_2d(st, &tm_x, bar_full(stage), kb * kBlockK, row0);
          ptx::tma_load_3d(st + kPfATile, &tm_w, bar_full(stage), kb * kBlockK, ch0, it.e);
          ptx::tma_load_3d(st + kPfATile + kWTileBytes, &tm_w, bar_full(stage), kb * kBlockK, ch1, it.e);
          ++arms;
          if (++stage == kPfStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        for (int s = 0; s < kPfStages; ++s) {
          const long long a = arms / kPfStages + (s < arms % kPfStages ? 1 : 0);
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
      constexpr uint32_t idesc = ptx::idesc_i8(kPfTokens, kPfCols);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
        const int nvalid = min(kPfTokens, s_start[it.e + 1] - (s_start[it.e] + it.tt * kPfTokens));
        const bool narrow = nvalid <= kPfNarrowMax;
        const uint32_t idesc_n = ptx::idesc_i8(128, (nvalid + 15) & ~15);
        if (!bounded_wait(bar_tempty(buf), tphase ^ 1u, s_abort, 12, p.wait_cycles)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d = tmem_base + buf * kPfCols;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_full(stage), phase, s_abort, 13, p.wait_cycles)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t st = tiles_addr + stage * kPfStageBytes;
          const uint64_t a = ptx::smem_desc_k128(st);
          const uint64_t b = ptx::smem_desc_k128(st + kPfATile);
          if (!narrow) {
#pragma unroll
            for (int k = 0; k < kBlockK / 32; ++k) ptx::mma_i8(d, a + 2 * k, b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          } else {
            const uint64_t b1 = ptx::smem_desc_k128(st + kPfATile + kWTileBytes);   // second 128 channels of the weight tile
#pragma unroll
            for (int k = 0; k < kBlockK / 32; ++k) {
              ptx::mma_i8(d, b + 2 * k, a + 2 * k, idesc_n, (kb | k) != 0 ? 1u : 0u);
              ptx::mma_i8(d + 128, b1 + 2 * k, a + 2 * k, idesc_n, (kb | k) != 0 ? 1u : 0u);
            }
          }
          ptx::mma_commit(bar_empty(stage));
          if (++stage == kPfStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit(bar_tfull(buf));
        if (++buf == kPfBufs) { buf = 0; tphase ^= 1u; }
      }
      if (!ok) {
        ptx::mma_commit(bar_drain);
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(bar_drain, 0) && clock64() - t0 < p.wait_cycles) {}
      }
    }
  } else {
    // ---------------- epilogue: warps 2..9, thread = token row, two warps split the columns of a row ----------------
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;          // TMEM lane = token row inside the tile
    const int et = threadIdx.x - 64;                  // 0..255 among the epilogue threads
    const int chalf = (warp - 2) >> 2;                // which half of the tile's columns this warp handles
    int buf = 0;
    uint32_t tphase = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x) {
      const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
      // weight scales of this tile's 256 columns -> shared memory (independent of the accumulators)
      float* ws = s_wscale + buf * kPfCols;
      {
        const int c_first = FUSED ? it.ct * 128 : it.ct * 256;
        const int c_second = FUSED ? p.half + it.ct * 128 : it.ct * 256 + 128;
        const int lim_first = FUSED ? p.half : p.N;
        const float* wrow = p.w_scale ? p.w_scale + static_cast<int64_t>(it.e) * p.N : nullptr;
        if (et < 128) ws[et] = (wrow && c_first + et < lim_first) ? wrow[c_first + et] : 1.f;
        else ws[et] = (wrow && c_second + et - 128 < p.N) ? wrow[c_second + et - 128] : 1.f;
      }
      if (et == 0) s_got[buf] = bounded_wait(bar_tfull(buf), tphase, s_abort, 14, p.wait_cycles) ? 1 : 0;
      epilogue_bar_sync();
      if (!s_got[buf]) break;
      ptx::tc_fence_after();
      const int row = s_start[it.e] + it.tt * kPfTokens + r_local;
      const bool rvalid = row < s_start[it.e + 1];
      const float ts = (rvalid && p.tok_scale) ? p.tok_scale[row] : 1.f;
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kPfCols;
      const int tile_row0 = s_start[it.e] + it.tt * kPfTokens;
      const int nvalid = min(kPfTokens, s_start[it.e + 1] - tile_row0);
      if (nvalid <= kPfNarrowMax) {
        pf_narrow_epilogue<FUSED>(p, it, ws, t0, tile_row0, nvalid, r_local, lane, chalf);
      } else if constexpr (FUSED) {
        const int cg0 = it.ct * 128;
        float amax = 0.f;
        float* hrow = p.h_out + static_cast<int64_t>(row) * p.half + cg0;
#pragma unroll 1
        for (int c = chalf * 64; c < chalf * 64 + 64; c += 16) {
          int g[16], u[16];
          __syncwarp();
          ptx::tmem_ld16(t0 + c, g);
          ptx::tmem_ld16(t0 + 128 + c, u);
          ptx::tmem_ld_wait();
          float h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float gv = __fmul_rn(__fmul_rn(__int2float_rn(g[j]), ts), ws[c + j]);
            const float uv = __fmul_rn(__fmul_rn(__int2float_rn(u[j]), ts), ws[128 + c + j]);
            h[j] = silu_mul(p.activate_left ? gv : uv, p.activate_left ? uv : gv);   // one SwiGLU, operands picked first
          }
          if (rvalid) {
            if (cg0 + c + 16 <= p.half) {
#pragma unroll
              for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(h[j]));
#pragma unroll
              for (int j = 0; j < 16; j += 4) __stcs(reinterpret_cast<float4*>(hrow + c + j), make_float4(h[j], h[j + 1], h[j + 2], h[j + 3]));
            } else {
              for (int j = 0; j < 16; ++j)
                if (cg0 + c + j < p.half) {
                  amax = fmaxf(amax, fabsf(h[j]));
                  hrow[c + j] = h[j];
                }
            }
          }
        }
        if (rvalid) atomicMax(p.amax + row, __float_as_uint(amax));
      } else {
        const int c0 = it.ct * 256;
        const bool vec_ok = (p.N & 7) == 0;
        if (p.out_dtype != TAB_I32 && vec_ok) {
          // 16-bit output: 32 columns at a time go through a per-warp shared-memory patch so that global stores
          // are 64-byte row segments (four lanes per row) instead of one 16-byte piece per lane and row.
          uint8_t* patch = s_out + (warp - 2) * 32 * kPfOutPitch;
          const int row_base = s_start[it.e] + it.tt * kPfTokens + quarter * 32;
          const int row_end = s_start[it.e + 1];
          const int esz = 2;
#pragma unroll 1
          for (int c = chalf * 128; c < chalf * 128 + 128; c += 32) {
            int a[16], b[16];
            __syncwarp();                              // the loads below are warp-collective; the patch is free again
            ptx::tmem_ld16(t0 + c, a);
            ptx::tmem_ld16(t0 + c + 16, b);
            ptx::tmem_ld_wait();
            if (p.bias != nullptr) {                   // uniform: the same bias entry for every lane (token rows), a broadcast load
              const int* brow = p.bias + static_cast<int64_t>(it.e) * p.N + c0 + c;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                a[j] += c0 + c + j < p.N ? __ldg(brow + j) : 0;
                b[j] += c0 + c + 16 + j < p.N ? __ldg(brow + 16 + j) : 0;
              }
            }
            float f[32];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              f[j] = __fmul_rn(__fmul_rn(__int2float_rn(a[j]), ts), ws[c + j]);
              f[16 + j] = __fmul_rn(__fmul_rn(__int2float_rn(b[j]), ts), ws[c + 16 + j]);
            }
            uint4* prow = reinterpret_cast<uint4*>(patch + lane * kPfOutPitch);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint4 v;
              if (p.out_dtype == TAB_BF16) {
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(f[8 * k + 2 * i], f[8 * k + 2 * i + 1]);
              } else {
                __half2* h2 = reinterpret_cast<__half2*>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) h2[i] = __floats2half2_rn(f[8 * k + 2 * i], f[8 * k + 2 * i + 1]);
              }
              prow[k] = v;
            }
            __syncwarp();
            const int piece = lane & 3;                // 16-byte piece of the 64-byte row segment
            const bool cvalid = c0 + c + piece * 8 < p.N;
#pragma unroll
            for (int it8 = 0; it8 < 4; ++it8) {
              const int r = it8 * 8 + (lane >> 2);
              const int grow = row_base + r;
              if (grow < row_end && cvalid) {
                const uint4 v = *reinterpret_cast<const uint4*>(patch + r * kPfOutPitch + piece * 16);
                uint8_t* orow = out_row_ptr(p, grow, esz);
                if (orow != nullptr)                      // a null table entry = no destination for this row
                  __stcs(reinterpret_cast<uint4*>(orow + static_cast<int64_t>(c0 + c) * esz + piece * 16), v);   // streamed: outputs must not push weights and rows out of L2
              }
            }
          }
        } else {
#pragma unroll 1
        for (int c = chalf * 128; c < chalf * 128 + 128; c += 16) {
          int a[16];
          __syncwarp();                                // the loads below are warp-collective
          ptx::tmem_ld16(t0 + c, a);
          ptx::tmem_ld_wait();
          if (p.bias != nullptr) {
            const int* brow = p.bias + static_cast<int64_t>(it.e) * p.N + c0 + c;
#pragma unroll
            for (int j = 0; j < 16; ++j) a[j] += c0 + c + j < p.N ? __ldg(brow + j) : 0;
          }
          if (rvalid && c0 + c < p.N) {
            if (p.out_dtype == TAB_I32) {
              int* o = static_cast<int*>(p.out) + static_cast<int64_t>(row) * p.N + c0 + c;
              if (c0 + c + 16 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) *reinterpret_cast<int4*>(o + j) = make_int4(a[j], a[j + 1], a[j + 2], a[j + 3]);
              } else {
                for (int j = 0; j < 16; ++j)
                  if (c0 + c + j < p.N) o[j] = a[j];
              }
            } else {
              uint8_t* orow = out_row_ptr(p, row, 2);
              for (int j = 0; j < 16 && orow != nullptr; ++j) {
                if (c0 + c + j >= p.N) break;
                const float f = __fmul_rn(__fmul_rn(__int2float_rn(a[j]), ts), ws[c + j]);
                if (p.out_dtype == TAB_BF16) reinterpret_cast<__nv_bfloat16*>(orow)[c0 + c + j] = __float2bfloat16_rn(f);
                else reinterpret_cast<__half*>(orow)[c0 + c + j] = __float2half_rn(f);
              }
            }
          }
        }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));
      if (++buf == kPfBufs) { buf = 0; tphase ^= 1u; }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<kPfBufs * kPfCols>(tmem_base);
  }
}

}  // namespace tab
