// Row streaming for the HBM-bound row kernels: whole rows travel from global memory into a ring of shared-memory
// stages by bulk asynchronous copies (cp.async.bulk with mbarrier completion, the untiled form of TMA), issued by one
// thread up to STAGES rows ahead of the row the CTA is working on.  The arithmetic of a row then never waits for its
// own loads, registers hold no row between passes (a second pass re-reads shared memory), and a persistent CTA keeps
// STAGES - 1 rows in flight at all times.
#pragma once

#include "ptx_sm100.cuh"
#include "tab_common.cuh"

namespace tab {

// Global -> shared bulk copy of `bytes` (multiple of 16; both addresses 16-byte aligned), completion counted in bytes
// on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

constexpr unsigned kRowWaitSpins = 1u << 28;   // bound of a stage wait (seconds); a healthy copy lands within microseconds

// Ring of STAGES row buffers.  Usage by all threads of the CTA, for its rows r_k = first + k * stride (k = 0, 1, ...):
//   RowRing<STAGES> ring(stage_base, bars, row_bytes, stage_pitch);           // then __syncthreads()
//   ring.prime(src_of_row, first, stride, rows);                               // fills every stage
//   for k: if (!ring.wait(k)) break; ... read ring.stage(k) ...; __syncthreads(); ring.refill(k, src_of_row, ...);
template <int STAGES>
struct RowRing {
  uint32_t base, bars, row_bytes, pitch;

  __device__ __forceinline__ RowRing(void* stage_base, uint64_t* bar_mem, uint32_t row_bytes_, uint32_t pitch_)
      : base(ptx::smem_u32(stage_base)), bars(ptx::smem_u32(bar_mem)), row_bytes(row_bytes_), pitch(pitch_) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; ++s) ptx::mbar_init(bars + 8u * s, 1);
      ptx::fence_barrier_init();
    }
  }

  __device__ __forceinline__ void issue(int k, const void* src) const {
    const int s = k % STAGES;
    ptx::mbar_expect_tx(bars + 8u * s, row_bytes);
    bulk_load(base + s * pitch, src, row_bytes, bars + 8u * s);
  }

  // Waits for the copy of ring slot k; false if the wait ran out (the caller records it and stops).
  __device__ __forceinline__ bool wait(int k) const {
    const uint32_t bar = bars + 8u * (k % STAGES), parity = static_cast<uint32_t>(k / STAGES) & 1u;
    unsigned spins = 0;
    while (!ptx::mbar_try_wait(bar, parity))
      if (++spins > kRowWaitSpins) return false;
    return true;
  }

  __device__ __forceinline__ uint32_t stage_offset(int k) const { return static_cast<uint32_t>(k % STAGES) * pitch; }
};

}  // namespace tab
