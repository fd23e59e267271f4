// Expert-parallel exchange over peer memory (NVLink / NVSwitch) for GPUs of one node.
//
// Dispatch and combine move rows with plain stores into the destination GPU's receive buffer (peer-mapped symmetric
// memory) instead of a library collective: no host read of the split sizes, every step is a kernel on the caller's
// stream, so a whole expert-parallel layer can live in one CUDA graph.  Remote memory is only ever WRITTEN from here,
// with ordinary st.global; everything a later kernel reads (TMA loads of the GEMM included) is local memory.
//
// Buffers of rank r (all inside one symmetric allocation, same offsets on every rank):
//   recv   [R sources][C rows][row_bytes + 16]   dispatch rows; the 16-byte tail holds the fp32 activation scale
//   counts [R sources][E_l]  int32               rows per local expert sent by each source
//   ret    [R owners][C rows][row_bytes]         expert outputs coming back, at the sender's own send positions
//   flags  4 x [R] uint64                        arrival / consumption counters written by the peers
// C = T * min(E_l, K) is the most rows one rank can send to another.
//
// Hand-over: a sender signals "data n is there" by storing n into its slot of the receiver's flag array after the
// data kernel (stream order + __threadfence_system + a release store); the receiver's wait kernel spins, bounded, with
// acquire loads.  The receiver acknowledges after it has copied the rows out, and a sender waits for the previous
// acknowledgement before it overwrites a peer's buffer.  Counters live on the device so that a replayed CUDA graph
// keeps counting.  A wait that runs out of time records a code in the status word and lets the stream continue.
#include <stdlib.h>

#include "tab_common.cuh"

namespace tab {

constexpr int kEpMaxRanks = 64;
constexpr int kEpMaxExperts = 2048;   // R * E_l of one exchange

// Bound of a flag wait in SM clock ticks: TAB_EP_WAIT_MS from the environment (read once), default 2000 ms.  Ranks are
// aligned by a host barrier when the buffers are created, so a healthy peer answers within microseconds.
static long long ep_wait_cycles() {
  static const long long cycles = []() {
    long long ms = 2000;
    if (const char* f = getenv("TAB_EP_WAIT_MS")) {
      const long long v = atoll(f);
      if (v >= 1 && v <= 600000) ms = v;
    }
    return ms * 2000000LL;
  }();
  return cycles;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One thread per peer stores the next sequence number into that peer's flag slot for this rank.
__global__ void ep_signal_kernel(unsigned long long* const* __restrict__ peer_flags, unsigned long long* counter, int R) {
  __shared__ unsigned long long s_value;
  if (threadIdx.x == 0) s_value = *counter + 1;
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < R) st_release_sys(peer_flags[threadIdx.x], s_value);
  __syncthreads();
  if (threadIdx.x == 0) *counter = s_value;
}

// Waits until every source's flag has reached the expected sequence number.  pre_increment = 1: expect counter + 1
// (new data); 0: expect the current counter (acknowledgement of the previous exchange).  The counter advances either way.
__global__ void ep_wait_kernel(const unsigned long long* __restrict__ flags, unsigned long long* counter, int R,
                               int pre_increment, int* status, int code, long long limit) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned long long expect = *counter + (pre_increment ? 1ull : 0ull);
  if (threadIdx.x < R) {
    const long long t0 = clock64();
    while (ld_acquire_sys(flags + threadIdx.x) < expect) {
      if (clock64() - t0 > limit) {
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_fail) atomicCAS(status, 0, code);
    *counter = *counter + 1;
  }
}

// First sorted position of every destination rank's rows, from the per-expert counts (E = R * E_l entries): one warp
// per destination sums that rank's counts with coalesced loads and a shuffle reduction.
__device__ __forceinline__ void rank_bases_to_smem(const int32_t* __restrict__ expert_counts, int R, int E_l, int* s_base) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int r = warp; r < R; r += nwarps) {
    int c = 0;
    for (int e = lane; e < E_l; e += 32) c += max(expert_counts[r * E_l + e], 0);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if (lane == 0) s_base[r + 1] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_base[0] = 0;
    for (int r = 0; r < R; ++r) s_base[r + 1] += s_base[r];
  }
  __syncthreads();
}

__device__ __forceinline__ int rank_of_position(const int* s_base, int R, int p) {
  int d = 0;
  while (d + 1 < R && s_base[d + 1] <= p) ++d;
  return d;
}

constexpr int kEpThreads = 128;

// Sender: row p of the expert-sorted send buffer goes to slot [my_rank][p - base(d)] of rank d's receive buffer.
// CTA 0 also delivers the per-expert counts, and every pair index f gets its slot position for the combine.
__global__ void __launch_bounds__(kEpThreads) ep_send_kernel(const uint4* __restrict__ rows, const float* __restrict__ scales,
                                                            const int32_t* __restrict__ expert_counts,
                                                            const int32_t* __restrict__ expand_idx, int R, int E_l, int C,
                                                            int vec_per_row, int M, int my_rank,
                                                            uint8_t* const* __restrict__ peer_recv,
                                                            int32_t* const* __restrict__ peer_counts,
                                                            int32_t* __restrict__ expand_idx_slot, int* status, int code,
                                                            const unsigned long long* __restrict__ ack_flags,
                                                            const unsigned long long* __restrict__ ack_counter,
                                                            long long limit, int ack_code) {
  __shared__ int s_base[kEpMaxRanks + 1];
  if (ack_flags != nullptr && threadIdx.x < R) {
    // the peers have copied the rows of the previous exchange out of their buffers (every CTA checks before it
    // stores; the counter is advanced by the hand-over kernel that follows this one)
    const unsigned long long expect = *ack_counter;
    const long long t0 = clock64();
    while (ld_acquire_sys(ack_flags + threadIdx.x) < expect) {
      if (clock64() - t0 > limit) {
        atomicCAS(status, 0, ack_code);
        break;
      }
    }
  }
  rank_bases_to_smem(expert_counts, R, E_l, s_base);
  const int64_t slot_bytes = static_cast<int64_t>(vec_per_row + 1) * 16;
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < R * E_l; i += kEpThreads) {
      const int d = i / E_l, e = i - d * E_l;
      peer_counts[d][my_rank * E_l + e] = max(expert_counts[i], 0);
    }
  }
  const int total = min(M, s_base[R]);     // pairs that were dropped before the sort have no row
  for (int p = blockIdx.x; p < total; p += gridDim.x) {
    const int d = rank_of_position(s_base, R, p);
    if (p - s_base[d] >= C) {           // more rows for one destination than its slot holds (counts and C disagree): not sent
      if (threadIdx.x == 0) atomicCAS(status, 0, code);
      continue;
    }
    uint8_t* slot = peer_recv[d] + (static_cast<int64_t>(my_rank) * C + (p - s_base[d])) * slot_bytes;
    copy_row16<kEpThreads>(reinterpret_cast<uint4*>(slot), rows + static_cast<int64_t>(p) * vec_per_row, vec_per_row);
    if (threadIdx.x == 0) {
      const float sc = scales ? scales[p] : 0.f;
      *reinterpret_cast<uint4*>(slot + static_cast<int64_t>(vec_per_row) * 16) = make_uint4(__float_as_uint(sc), 0u, 0u, 0u);
    }
  }
  for (int f = blockIdx.x * kEpThreads + threadIdx.x; f < M; f += gridDim.x * kEpThreads) {
    const int p = expand_idx[f];
    const int d = rank_of_position(s_base, R, p < 0 ? 0 : p);
    expand_idx_slot[f] = p < 0 ? -1 : d * C + (p - s_base[d]);
  }
}

__device__ __forceinline__ int ep_last_le(const int32_t* __restrict__ off, int lo, int hi, int i) {
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (off[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

// Receiver: slot records -> rows in (local expert, source rank) order plus their scales.  plan as written by
// tab_moe_exchange_plan with slot_rows = C.
__global__ void __launch_bounds__(kEpThreads) ep_unpack_kernel(const uint8_t* __restrict__ recv, const int32_t* __restrict__ plan,
                                                              int R, int E_l, int vec_per_row, int64_t dst_rows, int zero_fill,
                                                              uint4* __restrict__ dst, float* __restrict__ dst_scales) {
  const int n = R * E_l;
  const int32_t* wire_off = plan;
  const int32_t* exp_off = plan + n;
  const int total = exp_off[n];
  const int64_t slot_bytes = static_cast<int64_t>(vec_per_row + 1) * 16;
  for (int64_t i = blockIdx.x; i < dst_rows; i += gridDim.x) {
    uint4* dp = dst + i * vec_per_row;
    if (i < total) {
      const int b = ep_last_le(exp_off, 0, n, static_cast<int>(i));   // b = e*R + s
      const int e = b / R, s = b - e * R;
      const uint8_t* rec = recv + (static_cast<int64_t>(wire_off[s * E_l + e]) + (i - exp_off[b])) * slot_bytes;
      copy_row16<kEpThreads>(dp, reinterpret_cast<const uint4*>(rec), vec_per_row);
      if (threadIdx.x == 0) dst_scales[i] = *reinterpret_cast<const float*>(rec + static_cast<int64_t>(vec_per_row) * 16);
    } else if (zero_fill) {
      for (int v = threadIdx.x; v < vec_per_row; v += kEpThreads) dp[v] = make_uint4(0, 0, 0, 0);
      if (threadIdx.x == 0) dst_scales[i] = 0.f;
    }
  }
}

// Expert side of combine: row i of the (expert, source) ordered outputs returns to slot [my_rank][its send offset] of
// the source rank's return buffer.
__global__ void __launch_bounds__(kEpThreads) ep_return_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ plan, int R,
                                                              int E_l, int C, int vec_per_row, int my_rank,
                                                              uint8_t* const* __restrict__ peer_ret) {
  const int n = R * E_l;
  const int32_t* wire_off = plan;
  const int32_t* exp_off = plan + n;
  const int total = exp_off[n];
  for (int i = blockIdx.x; i < total; i += gridDim.x) {
    const int b = ep_last_le(exp_off, 0, n, i);
    const int e = b / R, s = b - e * R;
    const int within = wire_off[s * E_l + e] - s * C + (i - exp_off[b]);
    if (within < 0 || within >= C) continue;   // a plan that does not fit the slots: the row has no place, nothing is stored
    uint8_t* dstp = peer_ret[s] + (static_cast<int64_t>(my_rank) * C + within) * vec_per_row * 16;
    copy_row16<kEpThreads>(reinterpret_cast<uint4*>(dstp), y + static_cast<int64_t>(i) * vec_per_row, vec_per_row);
  }
}

// Address of every expert-output row in its source rank's return buffer (the rows that ep_return_kernel would copy
// there), for a GEMM epilogue that stores its output rows straight into peer memory.  Rows past the total get 0.
__global__ void __launch_bounds__(256) ep_return_plan_kernel(const int32_t* __restrict__ plan, int R, int E_l, int C,
                                                            int64_t row_bytes, int my_rank, int64_t max_rows,
                                                            uint8_t* const* __restrict__ peer_ret,
                                                            unsigned long long* __restrict__ row_dst) {
  const int n = R * E_l;
  const int32_t* wire_off = plan;
  const int32_t* exp_off = plan + n;
  const int total = exp_off[n];
  for (int64_t i = blockIdx.x * 256LL + threadIdx.x; i < max_rows; i += gridDim.x * 256LL) {
    unsigned long long a = 0ull;
    if (i < total) {
      const int b = ep_last_le(exp_off, 0, n, static_cast<int>(i));
      const int e = b / R, s = b - e * R;
      const int within = wire_off[s * E_l + e] - s * C + (static_cast<int>(i) - exp_off[b]);
      if (within >= 0 && within < C)    // else the plan does not fit the slots: the row keeps address 0 and is not stored
        a = reinterpret_cast<unsigned long long>(peer_ret[s] + (static_cast<int64_t>(my_rank) * C + within) * row_bytes);
    }
    row_dst[i] = a;
  }
}

// ---- fused forms: fewer launches per exchange ------------------------------------------------------------------

// Signal "my data is there" to every peer, then wait until every peer's data is here: the two one-CTA kernels of a
// hand-over in one.  bump (optional) is a second counter advanced by one: the acknowledgement counter that the data
// kernel before this one only read.
__global__ void ep_signal_wait_kernel(unsigned long long* const* __restrict__ peer_flags, unsigned long long* sig_counter,
                                      const unsigned long long* __restrict__ flags, unsigned long long* wait_counter, int R,
                                      int* status, int code, long long limit, unsigned long long* bump) {
  __shared__ unsigned long long s_value;
  __shared__ int s_fail;
  if (threadIdx.x == 0) {
    s_value = *sig_counter + 1;
    s_fail = 0;
  }
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < R) st_release_sys(peer_flags[threadIdx.x], s_value);
  const unsigned long long expect = *wait_counter + 1ull;
  if (threadIdx.x < R) {
    const long long t0 = clock64();
    while (ld_acquire_sys(flags + threadIdx.x) < expect) {
      if (clock64() - t0 > limit) {
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_fail) atomicCAS(status, 0, code);
    *sig_counter = s_value;
    *wait_counter = expect;
    if (bump != nullptr) *bump = *bump + 1;
  }
}

// Exclusive scan of vals[0..n) in shared memory by a CTA of THREADS threads (n <= 2048); returns the total.
// tmp holds THREADS / 32 + 1 ints.  Ends with a barrier.
template <int THREADS>
__device__ int cta_exclusive_scan(int* vals, int n, int* tmp) {
  const int per = (n + THREADS - 1) / THREADS;
  const int lo = threadIdx.x * per, hi = min(lo + per, n);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += vals[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) tmp[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int w = 0; w < THREADS / 32; ++w) {
      const int t = tmp[w];
      tmp[w] = run;
      run += t;
    }
    tmp[THREADS / 32] = run;
  }
  __syncthreads();
  int run = tmp[warp] + incl - sum;
  for (int i = lo; i < hi; ++i) {
    const int v = vals[i];
    vals[i] = run;
    run += v;
  }
  const int total = tmp[THREADS / 32];
  __syncthreads();
  return total;
}

// Row offsets of both sides of an exchange with fixed slots of C rows per source, in shared memory:
//   s_wire[s*E_l + e] = first slot row of the rows (source s, expert e);  s_exp[e*R + s] = first row of that block in
//   (expert, source) order, s_exp[R*E_l] = total.  count(s, e) is read through `at`.
template <int THREADS, typename CountAt>
__device__ __forceinline__ int build_exchange_offsets(CountAt at, int R, int E_l, int C, int* s_wire, int* s_exp, int* tmp) {
  const int n = R * E_l;
  for (int i = threadIdx.x; i < n; i += THREADS) {
    const int sr = i / E_l, e = i - sr * E_l;
    const int c = max(at(sr, e), 0);
    s_wire[i] = c;
    s_exp[e * R + sr] = c;
  }
  __syncthreads();
  cta_exclusive_scan<THREADS>(s_wire, n, tmp);
  const int total = cta_exclusive_scan<THREADS>(s_exp, n, tmp);
  // offset inside the source's fixed slot: subtract the source's first offset (read before anyone overwrites it)
  int first[(kEpMaxExperts + THREADS - 1) / THREADS];
  int k = 0;
  for (int i = threadIdx.x; i < n; i += THREADS, ++k) first[k] = s_wire[(i / E_l) * E_l];
  __syncthreads();
  k = 0;
  for (int i = threadIdx.x; i < n; i += THREADS, ++k) s_wire[i] = s_wire[i] - first[k] + (i / E_l) * C;
  if (threadIdx.x == 0) s_exp[n] = total;
  __syncthreads();
  return total;
}

// Receiver side of dispatch in one kernel: every CTA derives the row offsets from the delivered counts (a few hundred
// integers) and copies its share of the slot records into (local expert, source rank) order with their scales; CTA 0
// also writes expert_token_nums and ep_recv_count; the CTA that finishes last tells the peers that their rows have
// been copied out (the acknowledgement a sender checks before it overwrites the slots).
__global__ void __launch_bounds__(kEpThreads) ep_unpack_fused_kernel(const uint8_t* __restrict__ recv, const int32_t* __restrict__ counts,
                                                                    int R, int E_l, int C, int vec_per_row, int64_t dst_rows, int nums_type,
                                                                    uint4* __restrict__ dst, float* __restrict__ dst_scales,
                                                                    int64_t* __restrict__ expert_token_nums, int32_t* __restrict__ ep_recv_count,
                                                                    unsigned long long* const* __restrict__ ack_peer_flags,
                                                                    unsigned long long* ack_sig_counter, unsigned int* done_counter) {
  __shared__ int s_wire[kEpMaxExperts];
  __shared__ int s_exp[kEpMaxExperts + 1];
  __shared__ int s_tmp[kEpThreads / 32 + 1];
  __shared__ int s_last;
  const int n = R * E_l;
  const int total = build_exchange_offsets<kEpThreads>([&](int sr, int e) { return counts[sr * E_l + e]; }, R, E_l, C, s_wire, s_exp, s_tmp);
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < n; i += kEpThreads) {
      const int e = i / R, sr = i - e * R;
      ep_recv_count[i] = max(counts[sr * E_l + e], 0);
    }
    for (int e = threadIdx.x; e < E_l; e += kEpThreads) {
      const int begin = s_exp[e * R], end = e + 1 < E_l ? s_exp[(e + 1) * R] : total;
      expert_token_nums[e] = nums_type == 1 ? static_cast<int64_t>(end - begin) : static_cast<int64_t>(end);
    }
  }
  const int64_t slot_bytes = static_cast<int64_t>(vec_per_row + 1) * 16;
  const int64_t rows = total < dst_rows ? total : dst_rows;
  for (int64_t i = blockIdx.x; i < rows; i += gridDim.x) {
    const int b = ep_last_le(s_exp, 0, n, static_cast<int>(i));   // b = e*R + s
    const int e = b / R, sr = b - e * R;
    const uint8_t* rec = recv + (static_cast<int64_t>(s_wire[sr * E_l + e]) + (i - s_exp[b])) * slot_bytes;
    copy_row16<kEpThreads>(dst + i * vec_per_row, reinterpret_cast<const uint4*>(rec), vec_per_row);
    if (threadIdx.x == 0) dst_scales[i] = *reinterpret_cast<const float*>(rec + static_cast<int64_t>(vec_per_row) * 16);
  }
  if (ack_peer_flags != nullptr) {
    __syncthreads();                       // every thread's loads of the slots have returned (their stores were issued)
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = atomicInc(done_counter, gridDim.x - 1) == gridDim.x - 1 ? 1 : 0;   // wraps to 0 for the next launch
    }
    __syncthreads();
    if (s_last) {
      const unsigned long long v = *ack_sig_counter + 1;
      __syncthreads();
      if (threadIdx.x < R) st_release_sys(ack_peer_flags[threadIdx.x], v);
      if (threadIdx.x == 0) *ack_sig_counter = v;
    }
  }
}

// Expert side of combine in one kernel: every CTA derives the offsets from ep_send_counts (count of expert e from
// source s at e*R + s) and writes its share of the row address table (see ep_return_plan_kernel); CTA 0 also waits,
// bounded, until the sources have reduced the rows of the previous combine (the stores into their buffers come from
// the kernel launched after this one).
__global__ void __launch_bounds__(256) ep_return_plan_fused_kernel(const int32_t* __restrict__ ep_send_counts, int R, int E_l, int C,
                                                                  int64_t row_bytes, int my_rank, int64_t max_rows,
                                                                  uint8_t* const* __restrict__ peer_ret,
                                                                  unsigned long long* __restrict__ row_dst,
                                                                  const unsigned long long* __restrict__ ack_flags,
                                                                  unsigned long long* ack_counter, int* status, int ack_code,
                                                                  long long limit) {
  __shared__ int s_wire[kEpMaxExperts];
  __shared__ int s_exp[kEpMaxExperts + 1];
  __shared__ int s_tmp[256 / 32 + 1];
  const int n = R * E_l;
  const int total = build_exchange_offsets<256>([&](int sr, int e) { return ep_send_counts[e * R + sr]; }, R, E_l, C, s_wire, s_exp, s_tmp);
  for (int64_t i = blockIdx.x * 256LL + threadIdx.x; i < max_rows; i += gridDim.x * 256LL) {
    unsigned long long a = 0ull;
    if (i < total) {
      const int b = ep_last_le(s_exp, 0, n, static_cast<int>(i));
      const int e = b / R, sr = b - e * R;
      const int within = s_wire[sr * E_l + e] - sr * C + (static_cast<int>(i) - s_exp[b]);
      if (within >= 0 && within < C)
        a = reinterpret_cast<unsigned long long>(peer_ret[sr] + (static_cast<int64_t>(my_rank) * C + within) * row_bytes);
    }
    row_dst[i] = a;
  }
  if (blockIdx.x == 0 && ack_flags != nullptr) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    const unsigned long long expect = *ack_counter;
    if (threadIdx.x < R) {
      const long long t0 = clock64();
      while (ld_acquire_sys(ack_flags + threadIdx.x) < expect) {
        if (clock64() - t0 > limit) {
          s_fail = 1;
          break;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_fail) atomicCAS(status, 0, ack_code);
      *ack_counter = expect + 1;
    }
  }
}

}  // namespace tab

using namespace tab;

extern "C" int tab_ep_signal(void* const* peer_flags, void* counter, int64_t R, tab_stream_t stream) {
  if (!peer_flags || !counter || R < 1 || R > kEpMaxRanks) return fail(TAB_ERR_BAD_ARG, "ep_signal: bad argument (R=%lld)", (long long)R);
  ep_signal_kernel<<<1, 64, 0, as_stream(stream)>>>(reinterpret_cast<unsigned long long* const*>(peer_flags),
                                                   static_cast<unsigned long long*>(counter), (int)R);
  return check_launch("ep_signal");
}

extern "C" int tab_ep_wait(const void* flags, void* counter, int64_t R, int pre_increment, int* status, int code,
                           tab_stream_t stream) {
  if (!flags || !counter || !status || R < 1 || R > kEpMaxRanks) return fail(TAB_ERR_BAD_ARG, "ep_wait: bad argument (R=%lld)", (long long)R);
  ep_wait_kernel<<<1, 64, 0, as_stream(stream)>>>(static_cast<const unsigned long long*>(flags),
                                                 static_cast<unsigned long long*>(counter), (int)R, pre_increment, status, code,
                                                 ep_wait_cycles());
  return check_launch("ep_wait");
}

extern "C" int tab_ep_send_rows(const void* rows, const float* scales, const int32_t* expert_counts, const int32_t* expand_idx,
                                int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes, int64_t M, int64_t my_rank,
                                void* const* peer_recv, void* const* peer_counts, int32_t* expand_idx_slot,
                                int* status, int code, const void* ack_flags, const void* ack_counter, int ack_code,
                                tab_stream_t stream) {
  if (!expert_counts || !peer_recv || !peer_counts || !status || R < 1 || R > kEpMaxRanks || E_l < 1 || slot_rows < 1 || my_rank < 0 || my_rank >= R)
    return fail(TAB_ERR_BAD_ARG, "ep_send_rows: bad argument");
  if (M > 0 && (!rows || !expand_idx || !expand_idx_slot)) return fail(TAB_ERR_BAD_ARG, "ep_send_rows: null pointer");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || (M > 0 && !aligned16(rows)) || M > (1LL << 30) || R * slot_rows > (1LL << 30))
    return fail(TAB_ERR_ALIGNMENT, "ep_send_rows: row_bytes=%lld must be a multiple of 16, rows 16-byte aligned", (long long)row_bytes);
  const int grid = grid_for(M > 0 ? M : 1, 16);
  ep_send_kernel<<<grid, kEpThreads, 0, as_stream(stream)>>>(static_cast<const uint4*>(rows), scales, expert_counts, expand_idx, (int)R,
                                                            (int)E_l, (int)slot_rows, (int)(row_bytes / 16), (int)M, (int)my_rank,
                                                            reinterpret_cast<uint8_t* const*>(peer_recv),
                                                            reinterpret_cast<int32_t* const*>(peer_counts), expand_idx_slot, status, code,
                                                            static_cast<const unsigned long long*>(ack_flags),
                                                            static_cast<const unsigned long long*>(ack_counter), ep_wait_cycles(), ack_code);
  return check_launch("ep_send_rows");
}

extern "C" int tab_ep_unpack_rows(const void* recv, const int32_t* plan, int64_t R, int64_t E_l, int64_t row_bytes, int64_t dst_rows,
                                  int zero_fill, void* dst, float* dst_scales, tab_stream_t stream) {
  if (dst_rows == 0) return TAB_OK;
  if (!recv || !plan || !dst || !dst_scales || R < 1 || E_l < 1 || R * E_l > 2048 || dst_rows < 0 || dst_rows > (1LL << 30))
    return fail(TAB_ERR_BAD_ARG, "ep_unpack_rows: bad argument");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(recv) || !aligned16(dst))
    return fail(TAB_ERR_ALIGNMENT, "ep_unpack_rows: row_bytes=%lld must be a multiple of 16 and pointers 16-byte aligned", (long long)row_bytes);
  ep_unpack_kernel<<<grid_for(dst_rows, 16), kEpThreads, 0, as_stream(stream)>>>(static_cast<const uint8_t*>(recv), plan, (int)R, (int)E_l,
                                                                              (int)(row_bytes / 16), dst_rows, zero_fill,
                                                                              static_cast<uint4*>(dst), dst_scales);
  return check_launch("ep_unpack_rows");
}

extern "C" int tab_ep_return_rows(const void* y, const int32_t* plan, int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes,
                                  int64_t max_rows, int64_t my_rank, void* const* peer_ret, tab_stream_t stream) {
  if (max_rows == 0) return TAB_OK;
  if (!y || !plan || !peer_ret || R < 1 || R > kEpMaxRanks || E_l < 1 || R * E_l > 2048 || slot_rows < 1 || my_rank < 0 || my_rank >= R ||
      max_rows < 0 || max_rows > (1LL << 30))
    return fail(TAB_ERR_BAD_ARG, "ep_return_rows: bad argument");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(y))
    return fail(TAB_ERR_ALIGNMENT, "ep_return_rows: row_bytes=%lld must be a multiple of 16 and y 16-byte aligned", (long long)row_bytes);
  ep_return_kernel<<<grid_for(max_rows, 16), kEpThreads, 0, as_stream(stream)>>>(static_cast<const uint4*>(y), plan, (int)R, (int)E_l,
                                                                              (int)slot_rows, (int)(row_bytes / 16), (int)my_rank,
                                                                              reinterpret_cast<uint8_t* const*>(peer_ret));
  return check_launch("ep_return_rows");
}

extern "C" int tab_ep_return_plan(const int32_t* plan, int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes,
                                  int64_t max_rows, int64_t my_rank, void* const* peer_ret, uint64_t* row_dst,
                                  tab_stream_t stream) {
  if (max_rows == 0) return TAB_OK;
  if (!plan || !peer_ret || !row_dst || R < 1 || R > kEpMaxRanks || E_l < 1 || R * E_l > 2048 || slot_rows < 1 || my_rank < 0 ||
      my_rank >= R || max_rows < 0 || max_rows > (1LL << 30))
    return fail(TAB_ERR_BAD_ARG, "ep_return_plan: bad argument");
  if (row_bytes <= 0 || row_bytes % 16 != 0) return fail(TAB_ERR_ALIGNMENT, "ep_return_plan: row_bytes=%lld must be a multiple of 16", (long long)row_bytes);
  ep_return_plan_kernel<<<grid_for((max_rows + 255) / 256, 8), 256, 0, as_stream(stream)>>>(
      plan, (int)R, (int)E_l, (int)slot_rows, row_bytes, (int)my_rank, max_rows, reinterpret_cast<uint8_t* const*>(peer_ret),
      reinterpret_cast<unsigned long long*>(row_dst));
  return check_launch("ep_return_plan");
}

extern "C" int tab_ep_signal_wait(void* const* peer_flags, void* sig_counter, const void* flags, void* wait_counter, int64_t R,
                                  int* status, int code, void* bump_counter, tab_stream_t stream) {
  if (!peer_flags || !sig_counter || !flags || !wait_counter || !status || R < 1 || R > kEpMaxRanks)
    return fail(TAB_ERR_BAD_ARG, "ep_signal_wait: bad argument (R=%lld)", (long long)R);
  ep_signal_wait_kernel<<<1, 64, 0, as_stream(stream)>>>(reinterpret_cast<unsigned long long* const*>(peer_flags),
                                                        static_cast<unsigned long long*>(sig_counter),
                                                        static_cast<const unsigned long long*>(flags),
                                                        static_cast<unsigned long long*>(wait_counter), (int)R, status, code,
                                                        ep_wait_cycles(), static_cast<unsigned long long*>(bump_counter));
  return check_launch("ep_signal_wait");
}

extern "C" int tab_ep_unpack_rows_fused(const void* recv, const int32_t* recv_counts, int64_t R, int64_t E_l, int64_t slot_rows,
                                        int64_t row_bytes, int64_t dst_rows, int nums_type, void* dst, float* dst_scales,
                                        int64_t* expert_token_nums, int32_t* ep_recv_count, void* const* ack_peer_flags,
                                        void* ack_sig_counter, void* done_counter, tab_stream_t stream) {
  if (!recv || !recv_counts || !dst || !dst_scales || !expert_token_nums || !ep_recv_count || R < 1 || R > kEpMaxRanks || E_l < 1 ||
      R * E_l > kEpMaxExperts || slot_rows < 1 || dst_rows < 1 || dst_rows > (1LL << 30) || (nums_type != 0 && nums_type != 1))
    return fail(TAB_ERR_BAD_ARG, "ep_unpack_rows_fused: bad argument");
  if ((ack_peer_flags != nullptr) != (ack_sig_counter != nullptr) || (ack_peer_flags != nullptr) != (done_counter != nullptr))
    return fail(TAB_ERR_BAD_ARG, "ep_unpack_rows_fused: the acknowledgement needs its flags, its counter and the arrival counter");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(recv) || !aligned16(dst))
    return fail(TAB_ERR_ALIGNMENT, "ep_unpack_rows_fused: row_bytes=%lld must be a multiple of 16 and pointers 16-byte aligned", (long long)row_bytes);
  ep_unpack_fused_kernel<<<grid_for(dst_rows, 16), kEpThreads, 0, as_stream(stream)>>>(
      static_cast<const uint8_t*>(recv), recv_counts, (int)R, (int)E_l, (int)slot_rows, (int)(row_bytes / 16), dst_rows, nums_type,
      static_cast<uint4*>(dst), dst_scales, expert_token_nums, ep_recv_count,
      reinterpret_cast<unsigned long long* const*>(ack_peer_flags), static_cast<unsigned long long*>(ack_sig_counter),
      static_cast<unsigned int*>(done_counter));
  return check_launch("ep_unpack_rows_fused");
}

extern "C" int tab_ep_return_plan_fused(const int32_t* ep_send_counts, int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes,
                                        int64_t max_rows, int64_t my_rank, void* const* peer_ret, uint64_t* row_dst,
                                        const void* ack_flags, void* ack_counter, int* status, int ack_code, tab_stream_t stream) {
  if (max_rows == 0) return TAB_OK;
  if (!ep_send_counts || !peer_ret || !row_dst || R < 1 || R > kEpMaxRanks || E_l < 1 || R * E_l > kEpMaxExperts || slot_rows < 1 ||
      my_rank < 0 || my_rank >= R || max_rows < 0 || max_rows > (1LL << 30))
    return fail(TAB_ERR_BAD_ARG, "ep_return_plan_fused: bad argument");
  if ((ack_flags != nullptr) && (!ack_counter || !status)) return fail(TAB_ERR_BAD_ARG, "ep_return_plan_fused: the wait needs its counter and a status word");
  if (row_bytes <= 0 || row_bytes % 16 != 0) return fail(TAB_ERR_ALIGNMENT, "ep_return_plan_fused: row_bytes=%lld must be a multiple of 16", (long long)row_bytes);
  ep_return_plan_fused_kernel<<<grid_for((max_rows + 255) / 256, 4), 256, 0, as_stream(stream)>>>(
      ep_send_counts, (int)R, (int)E_l, (int)slot_rows, row_bytes, (int)my_rank, max_rows, reinterpret_cast<uint8_t* const*>(peer_ret),
      reinterpret_cast<unsigned long long*>(row_dst), static_cast<const unsigned long long*>(ack_flags),
      static_cast<unsigned long long*>(ack_counter), status, ack_code, ep_wait_cycles());
  return check_launch("ep_return_plan_fused");
}
