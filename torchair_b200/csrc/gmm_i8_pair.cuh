// Grouped int8 GEMM, prefill orientation on a CTA pair: two SMs of a cluster compute one 256-token x 256-channel tile
// with tcgen05.mma.cta_group::2.
//
// Why.  With a 128-token x 256-channel tile per CTA every unit of MMA work (one 128-byte K block) needs 48 KB of
// operands, and the tile stream is bound by the shared-memory fill rate (L2 -> SM) rather than by the tensor pipe.  On
// a pair each CTA loads its own 128 token rows and only HALF of the 256 weight channels; the MMA reads the other half
// out of the peer's shared memory.  Operand bytes per unit of MMA work fall to 32 KB, six stages fit instead of four,
// and every weight byte crosses L2 -> SM once per 256 tokens instead of once per 128.
//
// Layout.  CTA rank r of the pair (r = 0 leads) owns token rows [row0 + 128 r, +128) of the tile and its accumulator
// rows: 128 TMEM lanes x 256 columns (all channels), double-buffered.  Its half of the weight tile is
//   plain GEMM:    channels [256 ct + 128 r, +128)                 -> accumulator columns [128 r, +128)
//   fused gate_up: 64 gate channels [128 ct + 64 r, +64) followed by the matching 64 up channels
//                                                                   -> columns [128 r, +64) gate, [128 r + 64, +64) up
// so that gate and up of a channel meet in one thread of the epilogue, as in the single-CTA kernel.
//
// Protocol (all loads are ordinary, per-CTA TMA loads; nothing is multicast):
//   full[s]    lives in the leader; both CTAs' loads complete on it (cp.async.bulk.tensor .cta_group::2 lets a load
//              signal an mbarrier of the peer CTA); the leader's producer arms it for the bytes of both CTAs.
//   empty[s]   one per CTA; the leader's MMA warp commits to both (tcgen05.commit ... multicast::cluster).
//   tfull[b]   one per CTA, committed to both when a tile's MMAs are done; tempty[b] lives in the leader and counts the
//              epilogue warps of both CTAs (the peer's arrive remotely).
// Only the leader issues MMAs.  Tensor memory is allocated and released by each CTA with the cta_group::2 forms.
// Every wait is bounded as in the other kernels; a CTA that gives up records its code, skips to the end, and the final
// hand-shake between the two CTAs (each tells the other that it no longer touches the pair's shared state) is bounded
// too.
//
// Narrow tiles.  Tiles are 256 tokens; an expert's last tile with at most 64 rows (kPairNarrowMax) would waste nearly a
// whole tile of MMA work, so it is computed with the operands swapped, out of the same shared-memory stages: each CTA's
// half of the weight tile (128 rows) is its half of the 256-row operand, the tokens are the N operand with N = rows
// rounded up to 16, every CTA loading half of them.  An accumulator lane is then a channel and a column a token; the
// epilogue does the same arithmetic per element, so results do not depend on the form a tile took.  In the fused
// gate_up a CTA's lanes hold 64 gate channels followed by the 64 matching up channels: the up warps hand their
// dequantised values to the gate warps through shared memory.  Tails of 65..255 rows still cost a whole tile, so the host
// chooses this kernel where experts hold many rows or sit just above a multiple of 256 (see use_pair in gmm_i8.cu).
#pragma once

#include "gmm_common.cuh"
#include "gmm_i8_prefill.cuh"

namespace tab {

constexpr int kPairTokens = 256;                      // token rows per pair tile
constexpr int kPairStageBytes = kPfATile + kWTileBytes;   // 16 KB of tokens + 16 KB of weights per CTA
constexpr int kPairStages = 6;
constexpr int kPairNarrowMax = 64;                    // last tiles with at most this many rows swap the operands
static_assert(kPairNarrowMax * 64 * 4 <= kPfOutStageBytes, "the gate/up exchange of a narrow tile uses the output staging area");
constexpr int kPairSmemBytes = 1024 + kPairStages * kPairStageBytes + kPfCtrlBytes + kPfScaleBytes + kPfTableBytes + kPfOutStageBytes;
static_assert(kPairSmemBytes <= kSmemLimit, "pair GEMM shared memory");
static_assert(2 * kPairStages * 8 + 2 * kPfBufs * 8 + 16 <= 224, "barriers overflow the control block");

namespace ptx {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA tiled loads into this CTA's shared memory whose completion is counted on an mbarrier given by its
// shared::cluster address (it may belong to the peer CTA of the pair).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

template <int kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(kCols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(kCols) : "memory");
}

__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}

}  // namespace ptx

// Epilogue of a narrow tile on a pair (operands swapped): this thread's TMEM lane l is a channel of this CTA's half of the
// weight tile, columns are the tile's tokens (column j = row tile_start + j).  Plain: channel 256 ct + 128 rank + l.  Fused:
// lanes 0..63 hold gate channels 128 ct + 64 rank + l, lanes 64..127 the matching up channels; the up warps (lane quarters
// 2, 3) write their dequantised values to `xchg` [token][64], all eight warps meet, the gate warps finish.  The two warps
// of a lane quarter alternate over the 16-token column chunks.  Same arithmetic per element as the wide tiles.
template <bool FUSED>
__device__ __forceinline__ void pair_narrow_epilogue(const GmmParams& p, const WorkItem& it, const float* ws, uint32_t t0,
                                                     int tile_start, int nvalid, int rank, int quarter, int lane, int chalf,
                                                     float* xchg) {
  const int nv16 = (nvalid + 15) & ~15;
  const int l = quarter * 32 + lane;
  const float wv = ws[rank * 128 + l];
  if constexpr (FUSED) {
    const bool is_up = quarter >= 2;
    const int lc = l & 63;
    const int ch = it.ct * 128 + rank * 64 + lc;
    const bool cvalid = ch < p.half;
    if (is_up) {
#pragma unroll 1
      for (int c = chalf * 16; c < nv16; c += 32) {
        int u[16];
        __syncwarp();
        ptx::tmem_ld16(t0 + c, u);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool tvalid = c + j < nvalid;           // uniform over the warp
          const float ts = (tvalid && p.tok_scale) ? p.tok_scale[tile_start + c + j] : 1.f;
          xchg[(c + j) * 64 + lc] = __fmul_rn(__fmul_rn(__int2float_rn(u[j]), ts), wv);
        }
      }
    }
    epilogue_bar_sync();
    if (!is_up) {
#pragma unroll 1
      for (int c = chalf * 16; c < nv16; c += 32) {
        int g[16];
        __syncwarp();
        ptx::tmem_ld16(t0 + c, g);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool tvalid = c + j < nvalid;
          const int row = tile_start + c + j;
          const float ts = (tvalid && p.tok_scale) ? p.tok_scale[row] : 1.f;
          const float gv = __fmul_rn(__fmul_rn(__int2float_rn(g[j]), ts), wv);
          const float uv = xchg[(c + j) * 64 + lc];
          const float h = silu_mul(p.activate_left ? gv : uv, p.activate_left ? uv : gv);
          if (tvalid) {
            if (cvalid) __stcs(p.h_out + static_cast<int64_t>(row) * p.half + ch, h);
            const float m = warp_max(cvalid ? fabsf(h) : 0.f);
            if (lane == 0) atomicMax(p.amax + row, __float_as_uint(m));
          }
        }
      }
    }
  } else {
    const int ch = it.ct * 256 + rank * 128 + l;
    const bool cvalid = ch < p.N;
    const int bias = (cvalid && p.bias) ? p.bias[static_cast<int64_t>(it.e) * p.N + ch] : 0;
#pragma unroll 1
    for (int c = chalf * 16; c < nv16; c += 32) {
      int a[16];
      __syncwarp();
      ptx::tmem_ld16(t0 + c, a);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        a[j] += bias;
        const int row = tile_start + c + j;
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPfThreads, 1)
gmm_i8_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w64,
                   const __grid_constant__ CUtensorMap tm_x, const GmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t tiles_addr = ptx::smem_u32(smem);
  uint8_t* ctrl = smem + kPairStages * kPairStageBytes;
  const uint32_t bar0 = ptx::smem_u32(ctrl);
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kPairStages + s); };
  auto bar_tfull = [&](int b) { return bar0 + 8u * (2 * kPairStages + b); };
  auto bar_tempty = [&](int b) { return bar0 + 8u * (2 * kPairStages + kPfBufs + b); };
  const uint32_t bar_drain = bar0 + 8u * (2 * kPairStages + 2 * kPfBufs);
  const uint32_t bar_done = bar_drain + 8u;            // the peer no longer touches this CTA's shared state
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(ctrl + 224);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_got = reinterpret_cast<volatile int*>(s_tmem + 2);   // [2] outcome of the epilogue's wait, per buffer
  float* s_wscale = reinterpret_cast<float*>(ctrl + kPfCtrlBytes);     // [2][256]
  int* s_start = reinterpret_cast<int*>(ctrl + kPfCtrlBytes + kPfScaleBytes);
  int* s_pref = s_start + (kMaxGroups + 1);
  uint8_t* s_out = ctrl + kPfCtrlBytes + kPfScaleBytes + kPfTableBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int E = p.E;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(bar_full(s), 1);                      // armed by the leader's producer for the bytes of both CTAs
      ptx::mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < kPfBufs; ++b) {
      ptx::mbar_init(bar_tfull(b), 1);
      ptx::mbar_init(bar_tempty(b), 2 * kPfEpiWarps);      // epilogue warps of both CTAs
    }
    ptx::mbar_init(bar_drain, 1);
    ptx::mbar_init(bar_done, 1);
    *s_abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_w64);
    ptx::prefetch_tensormap(&tm_x);
  }
  if (warp == 1) ptx::tmem_alloc_pair<kPfBufs * kPfCols>(ptx::smem_u32(s_tmem));
  if (warp == 0) build_group_tables(p, kPairTokens, lane, s_start, s_pref);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync_all();          // both CTAs' barriers exist before anything signals across the pair
  ptx::tc_fence_after();

  const uint32_t tmem_base = *s_tmem;
  const int total_items = s_pref[E] * p.chan_tiles;
  const int num_kb = (p.Kd + kBlockK - 1) / kBlockK;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA): own 128 token rows + own half of the weight channels ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < total_items && ok; w += num_clusters) {
        const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
        const int tile_start = s_start[it.e] + it.tt * kPairTokens;
        const int nvalid = min(kPairTokens, s_start[it.e + 1] - tile_start);
        // narrow tile: the tokens are the N operand, this CTA brings half of them (the box still holds 128 rows)
        const int row0 = nvalid <= kPairNarrowMax ? tile_start + static_cast<int>(rank) * (((nvalid + 15) & ~15) >> 1)
                                                  : tile_start + static_cast<int>(rank) * kPfTokens;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_empty(stage), phase ^ 1u, s_abort, 21, p.wait_cycles)) { ok = false; break; }
          const uint32_t st = tiles_addr + stage * kPairStageBytes;
          const uint32_t full_leader = ptx::mapa(bar_full(stage), 0);
          if (leader) ptx::mbar_expect_tx(bar_full(stage), 2 * kPairStageBytes);
          ptx::tma_load_2d_pair(st, &tm_x, full_leader, kb * kBlockK, row0);
          if constexpr (FUSED) {
            const int g0 = it.ct * 128 + static_cast<int>(rank) * 64;
            ptx::tma_load_3d_pair(st + kPfATile, &tm_w64, full_leader, kb * kBlockK, g0, it.e);
            ptx::tma_load_3d_pair(st + kPfATile + 64 * kBlockK, &tm_w64, full_leader, kb * kBlockK, p.half + g0, it.e);
          } else {
            ptx::tma_load_3d_pair(st + kPfATile, &tm_w, full_leader, kb * kBlockK, it.ct * 256 + static_cast<int>(rank) * 128, it.e);
          }
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: the leader's warp, for both CTAs ----------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = ptx::idesc_i8(256, kPfCols);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int w = cluster_id; w < total_items && ok; w += num_clusters) {
        if (!bounded_wait(bar_tempty(buf), tphase ^ 1u, s_abort, 22, p.wait_cycles)) { ok = false; break; }
        ptx::tc_fence_after();
        const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
        const int nvalid = min(kPairTokens, s_start[it.e + 1] - (s_start[it.e] + it.tt * kPairTokens));
        const bool narrow = nvalid <= kPairNarrowMax;
        const uint32_t idesc_item = narrow ? ptx::idesc_i8(256, (nvalid + 15) & ~15) : idesc;
        const uint32_t d = tmem_base + buf * kPfCols;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bounded_wait(bar_full(stage), phase, s_abort, 23, p.wait_cycles)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t st = tiles_addr + stage * kPairStageBytes;
          const uint64_t tok = ptx::smem_desc_k128(st);
          const uint64_t wgt = ptx::smem_desc_k128(st + kPfATile);
          const uint64_t a = narrow ? wgt : tok;             // narrow: the weights are the 256-row operand
          const uint64_t b = narrow ? tok : wgt;
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k) ptx::mma_i8_pair(d, a + 2 * k, b + 2 * k, idesc_item, (kb | k) != 0 ? 1u : 0u);
          ptx::mma_commit_pair(bar_empty(stage));
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::mma_commit_pair(bar_tfull(buf));
        if (++buf == kPfBufs) { buf = 0; tphase ^= 1u; }
      }
      if (!ok) {
        ptx::mma_commit_pair(bar_drain);
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(bar_drain, 0) && clock64() - t0 < p.wait_cycles) {}
      }
    }
  } else {
    // ---------------- epilogue: warps 2..9, thread = token row, two warps split the columns of a row ----------------
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;
    const int et = threadIdx.x - 64;
    const int chalf = (warp - 2) >> 2;
    int buf = 0;
    uint32_t tphase = 0;
    for (int w = cluster_id; w < total_items; w += num_clusters) {
      const WorkItem it = decode_item(w, p.chan_tiles, E, s_pref);
      // weight scales of the tile's 256 accumulator columns -> shared memory
      float* ws = s_wscale + buf * kPfCols;
      {
        const float* wrow = p.w_scale ? p.w_scale + static_cast<int64_t>(it.e) * p.N : nullptr;
        int ch;
        bool in;
        if constexpr (FUSED) {                       // columns: [64 gate | 64 up] of CTA 0, then of CTA 1
          const int c = it.ct * 128 + (et >> 7) * 64 + (et & 63);
          in = c < p.half;
          ch = ((et >> 6) & 1) ? p.half + c : c;
        } else {
          ch = it.ct * 256 + et;
          in = ch < p.N;
        }
        ws[et] = (wrow && in) ? wrow[ch] : 1.f;
      }
      if (et == 0) s_got[buf] = bounded_wait(bar_tfull(buf), tphase, s_abort, 24, p.wait_cycles) ? 1 : 0;
      epilogue_bar_sync();
      if (!s_got[buf]) break;
      ptx::tc_fence_after();
      const int tile_start = s_start[it.e] + it.tt * kPairTokens;
      const int tile_row0 = tile_start + static_cast<int>(rank) * kPfTokens;
      const int row_end = s_start[it.e + 1];
      const int row = tile_row0 + r_local;
      const bool rvalid = row < row_end;
      const float ts = (rvalid && p.tok_scale) ? p.tok_scale[row] : 1.f;
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kPfCols;
      if (row_end - tile_start <= kPairNarrowMax) {
        pair_narrow_epilogue<FUSED>(p, it, ws, t0, tile_start, row_end - tile_start, static_cast<int>(rank), quarter, lane, chalf,
                                    reinterpret_cast<float*>(s_out));
      } else if (tile_row0 < row_end) {              // (a tile whose second half holds no rows leaves the peer nothing to store)
        if constexpr (FUSED) {
          // this warp takes the gate/up block of CTA `chalf`: accumulator columns [128 chalf, +64) and [128 chalf + 64, +64)
          const int cg0 = it.ct * 128 + chalf * 64;
          float amax = 0.f;
          float* hrow = p.h_out + static_cast<int64_t>(row) * p.half + cg0;
#pragma unroll 1
          for (int c = 0; c < 64; c += 16) {
            int g[16], u[16];
            __syncwarp();
            ptx::tmem_ld16(t0 + chalf * 128 + c, g);
            ptx::tmem_ld16(t0 + chalf * 128 + 64 + c, u);
            ptx::tmem_ld_wait();
            float h[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float gv = __fmul_rn(__fmul_rn(__int2float_rn(g[j]), ts), ws[chalf * 128 + c + j]);
              const float uv = __fmul_rn(__fmul_rn(__int2float_rn(u[j]), ts), ws[chalf * 128 + 64 + c + j]);
              h[j] = p.activate_left ? silu_mul(gv, uv) : silu_mul(uv, gv);
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
            uint8_t* patch = s_out + (warp - 2) * 32 * kPfOutPitch;
            const int row_base = tile_row0 + quarter * 32;
            const int esz = 2;
#pragma unroll 1
            for (int c = chalf * 128; c < chalf * 128 + 128; c += 32) {
              int a[16], b[16];
              __syncwarp();
              ptx::tmem_ld16(t0 + c, a);
              ptx::tmem_ld16(t0 + c + 16, b);
              ptx::tmem_ld_wait();
              if (p.bias != nullptr) {
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
              const int piece = lane & 3;
              const bool cvalid = c0 + c + piece * 8 < p.N;
#pragma unroll
              for (int it8 = 0; it8 < 4; ++it8) {
                const int r = it8 * 8 + (lane >> 2);
                const int grow = row_base + r;
                if (grow < row_end && cvalid) {
                  const uint4 v = *reinterpret_cast<const uint4*>(patch + r * kPfOutPitch + piece * 16);
                  uint8_t* orow = out_row_ptr(p, grow, esz);
                  if (orow != nullptr) __stcs(reinterpret_cast<uint4*>(orow + static_cast<int64_t>(c0 + c) * esz + piece * 16), v);
                }
              }
            }
          } else {
#pragma unroll 1
            for (int c = chalf * 128; c < chalf * 128 + 128; c += 16) {
              int a[16];
              __syncwarp();
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
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(bar_tempty(buf), 0));   // the leader counts both CTAs' warps
      if (++buf == kPfBufs) { buf = 0; tphase ^= 1u; }
    }
  }

  // End of the pair's work.  The peer may still read this CTA's shared memory (its MMAs) or signal its barriers until it
  // is through as well: tell the peer, wait (bounded) for the peer, then release tensor memory.
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::mbar_arrive_cluster(ptx::mapa(bar_done, rank ^ 1u));
    const long long t0 = clock64();
    while (!ptx::mbar_try_wait(bar_done, 0)) {
      if (clock64() - t0 > p.wait_cycles) {
        atomicCAS(&g_gmm_status, 0, 25);
        break;
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair<kPfBufs * kPfCols>(tmem_base);
  }
}

}  // namespace tab
