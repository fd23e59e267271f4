// Routing kernels of the MoE path: stable counting sort of (token, k) pairs by expert id
// (npu_moe_init_routing, sender side of npu_moe_distribute_dispatch), the fused quantise-and-scatter of
// token rows, the receiver-side row permutations around the all-to-all, and the weighted gather-sum of
// npu_moe_distribute_combine.  Integer/byte movers: HBM-bound, 16-byte accesses, grids sized to the SMs.
#include <mutex>

#include "row_pipe.cuh"
#include "tab_common.cuh"

namespace tab {

constexpr int kChunk = 1024;        // pairs per CTA in the sort kernels (32 warps x 32 lanes)
constexpr int kMaxExperts = 2048;   // bins of the counting sort

// Exclusive scan of vals[0..n) (n <= 2*blockDim.x, blockDim.x == 1024) in shared memory; returns the total.
__device__ int block_exclusive_scan(int* vals, int n, int* warp_sums) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int i0 = 2 * tid, i1 = 2 * tid + 1;
  const int a = i0 < n ? vals[i0] : 0;
  const int b = i1 < n ? vals[i1] : 0;
  int s = a + b;
  int incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sums[lane];
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sums[lane] = wi - w;  // exclusive
    if (lane == 31) warp_sums[32] = wi;
  }
  __syncthreads();
  const int excl = warp_sums[warp] + incl - s;
  if (i0 < n) vals[i0] = excl;
  if (i1 < n) vals[i1] = excl + a;
  const int total = warp_sums[32];
  __syncthreads();
  return total;
}

// Status word of the routing kernels on this device (tab_routing_status reads and clears it):
// bit 0 = an expert id outside [0, bound) was clamped, bit 1 = a row_idx value outside [0, T*K) was skipped,
// bit 2 = a bounded wait for a bulk copy gave up.
__device__ int g_routing_status = 0;

// Which (token, k) pairs take part in a sort and under which key.  Experts [lo, hi) are kept under key id - lo; the
// bin after them (key hi - lo, the last of nb = hi - lo + 1 bins) collects the pairs that are dropped: pairs of tokens
// whose mask byte is 0, and -- when drop_outside is set -- pairs whose expert lies outside the range (an expert range
// narrower than the model's, or special experts that are not dispatched).  Without drop_outside an id outside the
// range is clamped to the nearest kept expert and reported in the status word: no access goes out of range either way.
struct PairFilter {
  const uint8_t* mask;   // [T] or null
  int K;                 // pairs per token
  int lo, hi;
  int drop_outside;
};

__device__ __forceinline__ int pair_key(const PairFilter& pf, int id, int f) {
  const int dropped = pf.hi - pf.lo;
  if (pf.mask != nullptr && pf.mask[f / pf.K] == 0) return dropped;
  if (id >= pf.lo && id < pf.hi) return id - pf.lo;
  if (pf.drop_outside) return dropped;
  atomicOr(&g_routing_status, 1);
  return id < pf.lo ? 0 : dropped - 1;
}

// Phase 1: per-chunk histogram of expert ids.  chunk_hist [nchunks, nb].
__global__ void __launch_bounds__(kChunk) route_hist_kernel(const int32_t* __restrict__ expert, int n, int nb, const PairFilter pf,
                                                            int* __restrict__ chunk_hist) {
  extern __shared__ int s_hist[];
  for (int i = threadIdx.x; i < nb; i += kChunk) s_hist[i] = 0;
  __syncthreads();
  const int f = blockIdx.x * kChunk + threadIdx.x;
  if (f < n) atomicAdd(&s_hist[pair_key(pf, expert[f], f)], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < nb; i += kChunk) chunk_hist[blockIdx.x * nb + i] = s_hist[i];
}

// Phase 2: one warp per expert turns that expert's column of chunk_hist into an exclusive prefix over the chunks
// (in place) and writes the expert's total.  expert_count int32 [nb] (optional second copy out).
constexpr int kScanWarps = 8;
__global__ void __launch_bounds__(kScanWarps * 32) route_scan_kernel(int* __restrict__ chunk_hist, int nchunks, int nb,
                                                                    int* __restrict__ expert_count,
                                                                    int* __restrict__ expert_count_out, int nb_out) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * kScanWarps + (threadIdx.x >> 5);
  if (e >= nb) return;
  int run = 0;
  for (int c0 = 0; c0 < nchunks; c0 += 32) {
    const int c = c0 + lane;
    const int h = c < nchunks ? chunk_hist[c * nb + e] : 0;
    int incl = h;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (c < nchunks) chunk_hist[c * nb + e] = run + incl - h;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) {
    expert_count[e] = run;
    if (expert_count_out && e < nb_out) expert_count_out[e] = run;   // the bin of dropped pairs is not reported
  }
}

// Phase 3: stable rank of every pair inside its chunk (warp match + per-warp counts) plus the chunk base.
//   sorted_expert[pos] = key (expert id - lo), sorted_src[pos] = src_val[f] (or f when src_val is null),
//   inverse[inv_key] = pos where inv_key = src_val[f] (init_routing: expanded_row_idx is indexed by the
//   row_idx VALUE) or f (dispatch: expand_idx is indexed by the flattened pair index); -1 for a dropped pair.
__global__ void __launch_bounds__(kChunk) route_scatter_kernel(const int32_t* __restrict__ expert,
                                                               const int32_t* __restrict__ src_val, int n, int nb,
                                                               const PairFilter pf,
                                                               const int* __restrict__ chunk_base,
                                                               const int* __restrict__ expert_count,
                                                               int32_t* __restrict__ sorted_expert,
                                                               int32_t* __restrict__ sorted_src,
                                                               int32_t* __restrict__ inverse) {
  extern __shared__ unsigned short s_wcnt[];  // [32 warps][nb], then int s_base[nb]
  __shared__ int s_warp[33];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* s_base = reinterpret_cast<int*>(s_wcnt + 32 * nb);   // first row of every expert = exclusive scan of totals
  for (int i = tid; i < 32 * nb; i += kChunk) s_wcnt[i] = 0;
  for (int i = tid; i < nb; i += kChunk) s_base[i] = expert_count[i];
  __syncthreads();
  block_exclusive_scan(s_base, nb, s_warp);
  const int f = blockIdx.x * kChunk + tid;
  const bool valid = f < n;
  const int key = valid ? pair_key(pf, expert[f], f) : -1;
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (valid && rank_in_warp == 0) s_wcnt[warp * nb + key] = static_cast<unsigned short>(__popc(peers));
  __syncthreads();
  for (int e = tid; e < nb; e += kChunk) {  // exclusive prefix over the 32 warps, per expert column
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) {
      const int c = s_wcnt[w * nb + e];
      s_wcnt[w * nb + e] = static_cast<unsigned short>(run);
      run += c;
    }
  }
  __syncthreads();
  if (valid) {
    const int pos = s_base[key] + chunk_base[blockIdx.x * nb + key] + s_wcnt[warp * nb + key] + rank_in_warp;
    int sv = src_val ? src_val[f] : f;
    sorted_expert[pos] = key;
    if (sv < 0 || sv >= n) {            // a row_idx value that names no pair: nothing is written through it
      atomicOr(&g_routing_status, 2);
      sv = f;                            // the gather then reads the pair's own token instead of an arbitrary row
    } else {
      inverse[sv] = key == nb - 1 ? -1 : pos;
    }
    if (sorted_src) sorted_src[pos] = sv;
  }
}

struct SortScratch {
  int* chunk_hist;    // [nchunks, nb]
  int* expert_count;  // [nb]
  int32_t* sorted_src;     // [n]
  int32_t* sorted_expert;  // [n] (dispatch only; init_routing writes the caller's output)
};

static size_t sort_scratch_bytes(int64_t n, int64_t nb, bool need_sorted_expert) {
  const int64_t nchunks = (n + kChunk - 1) / kChunk;
  size_t ints = static_cast<size_t>(nchunks * nb + nb + 4 + n + (need_sorted_expert ? n : 0));
  return (ints * 4 + 255) / 256 * 256;
}

static SortScratch carve(void* ws, int64_t n, int64_t nb, bool need_sorted_expert) {
  const int64_t nchunks = (n + kChunk - 1) / kChunk;
  SortScratch s;
  int* p = static_cast<int*>(ws);
  s.chunk_hist = p; p += nchunks * nb;
  s.expert_count = p; p += nb;
  p += 4;   // spare words (keeps the following arrays 16-byte aligned when nb is a multiple of 4)
  s.sorted_src = p; p += n;
  s.sorted_expert = need_sorted_expert ? p : nullptr;
  return s;
}

// nb = pf.hi - pf.lo + 1 bins (the last one takes the dropped pairs); expert_count_out gets the nb - 1 kept experts.
static int run_sort(const int32_t* expert, const int32_t* src_val, int64_t n, const PairFilter& pf, const SortScratch& s,
                    int32_t* sorted_expert, int32_t* inverse, int32_t* expert_count_out, cudaStream_t st) {
  const int64_t nb = pf.hi - pf.lo + 1;
  const int nchunks = static_cast<int>((n + kChunk - 1) / kChunk);
  const size_t scatter_smem = static_cast<size_t>(32) * nb * sizeof(unsigned short) + static_cast<size_t>(nb) * sizeof(int);
  if (scatter_smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(route_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(scatter_smem));
    if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "routing: shared memory opt-in failed: %s", cudaGetErrorString(e));
  }
  route_hist_kernel<<<nchunks, kChunk, nb * sizeof(int), st>>>(expert, (int)n, (int)nb, pf, s.chunk_hist);
  route_scan_kernel<<<(int)((nb + kScanWarps - 1) / kScanWarps), kScanWarps * 32, 0, st>>>(s.chunk_hist, nchunks, (int)nb,
                                                                                          s.expert_count, expert_count_out, (int)nb - 1);
  route_scatter_kernel<<<nchunks, kChunk, scatter_smem, st>>>(expert, src_val, (int)n, (int)nb, pf, s.chunk_hist, s.expert_count,
                                                             sorted_expert, s.sorted_src, inverse);
  return check_launch("routing sort", 3);
}

// dst[i] = src[(idx[i] % mod)] for i < rows; one CTA per row, 16-byte vectors.
constexpr int kRowCopyThreads = 128;
__global__ void __launch_bounds__(kRowCopyThreads) gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ idx,
                                                                      int mod, int64_t rows, int vec_per_row,
                                                                      uint4* __restrict__ dst) {
  int64_t i = blockIdx.x;
  int next = i < rows ? idx[i] : 0;
  for (; i < rows; i += gridDim.x) {
    const int64_t s = (next < 0 ? 0 : next) % mod;
    if (i + gridDim.x < rows) next = idx[i + gridDim.x];   // fetched while this row is being copied
    copy_row16<kRowCopyThreads>(dst + i * vec_per_row, src + s * vec_per_row, vec_per_row);
  }
}

// Token-major form of the same gather for rows of 512 B .. 48 KB, moved entirely by the copy engine of the SM: a
// one-warp CTA streams its tokens' rows into a ring of shared-memory stages with bulk loads and sends every staged
// row to the K sorted positions of its copies with bulk stores (no register traffic, 16 KB per instruction).  The K
// copies of token t are the pairs whose row_idx value is t + j*T (value % T == t); inverse[value] is their position;
// positions at or past out_rows are dropped (active_num).
constexpr int kBulkStages = 4;
__global__ void __launch_bounds__(32) scatter_rows_bulk_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ inverse,
                                                               int64_t tokens, int K, int64_t out_rows, uint32_t row_bytes,
                                                               uint8_t* __restrict__ dst) {
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ uint64_t bars[kBulkStages];
  RowRing<kBulkStages> ring(ring_mem, bars, row_bytes, row_bytes);
  __syncwarp();
  const int lane = threadIdx.x;
  const int64_t first = blockIdx.x, stride = gridDim.x;
  if (lane == 0)
    for (int k = 0; k < kBulkStages; ++k)
      if (first + k * stride < tokens) ring.issue(k, x + (first + k * stride) * row_bytes);
  int k = 0;
  for (int64_t t = first; t < tokens; t += stride, ++k) {
    bool ok = true;
    for (int j0 = 0; j0 < K && ok; j0 += 32) {
      const int j = j0 + lane;
      const int pos = j < K ? inverse[t + static_cast<int64_t>(j) * tokens] : -1;   // in flight while the row lands
      if (j0 == 0) ok = __all_sync(0xffffffffu, ring.wait(k) ? 1 : 0) != 0;
      if (!ok) break;
      const int n = min(32, K - j0);
      for (int jj = 0; jj < n; ++jj) {      // lane 0 issues the stores; the positions come from the lanes that loaded them
        const int p = __shfl_sync(0xffffffffu, pos, jj);
        if (lane == 0 && p >= 0 && p < out_rows)
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dst + static_cast<int64_t>(p) * row_bytes), "r"(ring.base + ring.stage_offset(k)), "r"(row_bytes) : "memory");
      }
    }
    if (!ok) {                               // a row that never landed: report and stop (nothing was stored from its stage)
      if (lane == 0) atomicOr(&g_routing_status, 4);
      break;
    }
    if (lane == 0) {
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      // once the stores of the previous token have read their stage, it takes the row kBulkStages - 1 tokens ahead
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      if (k >= 1 && t + (kBulkStages - 1) * stride < tokens)
        ring.issue(k - 1 + kBulkStages, x + (t + (kBulkStages - 1) * stride) * row_bytes);
    }
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Sender side of dispatch: one CTA per token; quantise the row once (or copy it), then write the K copies
// to their sorted positions.  cols % 16 == 0.  The row stays in registers in raw form between the passes.
constexpr int kPackChunks = 8;
constexpr int kPackMaxK = 256;
constexpr int kSmallPairs = 4096;   // T*K up to which the sort runs inside the pack kernel (one launch instead of four)

// kSortInside = false: expand_idx holds the sorted position of every pair (written by the three sort kernels; -1 for
// a dropped pair) and counts the rows per expert.  kSortInside = true (T*K <= kSmallPairs): the kernel sorts by itself
// -- every CTA keeps the keys of ALL pairs in shared memory and ranks the K pairs of its token directly (position =
// pairs with a smaller key, plus earlier pairs with the same key: the stable order of the counting sort); the last CTA
// also builds the per-expert counts.  expand_idx, counts and sorted_src are then outputs, expert_ids the input.
// kSmooth (quantising only): every copy is quantised on its own after multiplying the row by the fp32 smooth-scale row
// of its expert (smooth [smooth_rows, cols]; one row for all experts when smooth_rows == 1).
struct PackArgs {
  int32_t* expand_idx;
  int64_t tokens;
  int K, cols;
  void* send_rows;
  float* send_scales;
  int32_t* counts;
  int64_t* nums64;
  int num_experts;      // kept experts = pf.hi - pf.lo
  int nums_type;
  const int32_t* expert_ids;
  int32_t* sorted_src;
  const float* smooth;
  int smooth_rows;
  const float* passthrough_scale;   // not quantising: per-token value copied to send_scales of every copy (or null: 0)
  int pos_limit;                    // copies at sorted positions >= pos_limit get no row (their indices are still reported)
  PairFilter pf;
};

template <typename T, bool kQuant, int THREADS, bool kSortInside, bool kSmooth>
__global__ void __launch_bounds__(THREADS) dispatch_pack_kernel(const T* __restrict__ x, const PackArgs a) {
  __shared__ float red[THREADS / 32];
  __shared__ int s_pos[kPackMaxK];
  __shared__ int s_key[kSmooth ? kPackMaxK : 1];
  __shared__ short s_e[kSortInside ? kSmallPairs : 1];
  __shared__ int s_hist[kSortInside ? kMaxExperts + 1 : 1];
  const int K = a.K, cols = a.cols, num_experts = a.num_experts;
  const int64_t tokens = a.tokens;
  const int nchunk = cols >> 3;
  // A row's loads do not depend on its positions: they are issued before the ranking so that their latency covers it (with
  // the sort inside, before the keys of all pairs are read; the first token of a CTA is then already on its way).
  Raw8<T> raw[kQuant ? kPackChunks : 1];
  auto load_row = [&](int64_t t) {
    if constexpr (kQuant) {
#pragma unroll
      for (int c = 0; c < kPackChunks; ++c) {
        const int ch = threadIdx.x + c * THREADS;
        if (ch < nchunk) raw[c].load(x + t * cols + ch * 8);
      }
    }
  };
  if constexpr (kSortInside) {
    if (blockIdx.x < tokens) load_row(blockIdx.x);
    const int n = static_cast<int>(tokens) * K;
    const bool last = blockIdx.x == gridDim.x - 1;
    if (last)
      for (int e = threadIdx.x; e <= num_experts; e += THREADS) s_hist[e] = 0;
    for (int f = threadIdx.x; f < n; f += THREADS) s_e[f] = static_cast<short>(pair_key(a.pf, a.expert_ids[f], f));
    __syncthreads();
    if (last) {
      for (int f = threadIdx.x; f < n; f += THREADS) atomicAdd(&s_hist[s_e[f]], 1);
      __syncthreads();
      for (int e = threadIdx.x; e < num_experts; e += THREADS) a.counts[e] = s_hist[e];
    }
  }
  if (a.nums64 != nullptr && blockIdx.x == gridDim.x - 1 && threadIdx.x < 32) {
    // the per-expert copies as int64 counts (nums_type 1) or their running total (0), the form the grouped GEMM reads
    long long run = 0;
    for (int e0 = 0; e0 < num_experts; e0 += 32) {
      const int e = e0 + threadIdx.x;
      const long long c = e < num_experts ? (kSortInside ? s_hist[e] : a.counts[e]) : 0;
      long long incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const long long t = __shfl_up_sync(0xffffffffu, incl, o);
        if (threadIdx.x >= o) incl += t;
      }
      if (e < num_experts) a.nums64[e] = a.nums_type == 1 ? c : run + incl;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    const T* xr = x + t * cols;
    if (kSortInside && t != blockIdx.x) load_row(t);
    __syncthreads();   // previous token's positions are no longer read
    if constexpr (kSortInside) {
      const int n = static_cast<int>(tokens) * K;
      const int lane = threadIdx.x & 31;
      for (int k = threadIdx.x >> 5; k < K; k += THREADS / 32) {     // one warp per pair of this token
        const int f0 = static_cast<int>(t) * K + k;
        const int e0 = s_e[f0];
        int before = 0;
        for (int f = lane; f < n; f += 32) {
          const int e = s_e[f];
          before += (e < e0 || (e == e0 && f < f0)) ? 1 : 0;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
        if (lane == 0) {
          if (a.sorted_src != nullptr) a.sorted_src[before] = f0;
          if (e0 == num_experts) before = -1;                         // dropped pair: no row
          a.expand_idx[f0] = before;
          s_pos[k] = before < a.pos_limit ? before : -1;
          if constexpr (kSmooth) s_key[k] = e0;
        }
      }
    } else {
      for (int k = threadIdx.x; k < K; k += THREADS) {
        const int p = a.expand_idx[t * K + k];
        s_pos[k] = p < a.pos_limit ? p : -1;
        if constexpr (kSmooth) s_key[k] = pair_key(a.pf, a.expert_ids[t * K + k], static_cast<int>(t) * K + k);
      }
    }
    __syncthreads();   // positions (and keys) are published
    if constexpr (kQuant) {
      if constexpr (!kSortInside) load_row(t);     // many tokens per CTA: the loads of a row directly before its arithmetic
      int8_t* out = static_cast<int8_t*>(a.send_rows);
      if constexpr (!kSmooth) {
        float amax = 0.f;
#pragma unroll
        for (int c = 0; c < kPackChunks; ++c) {
          const int ch = threadIdx.x + c * THREADS;
          if (ch < nchunk) amax = fmaxf(amax, raw_amax(raw[c]));
        }
        for (int ch = threadIdx.x + kPackChunks * THREADS; ch < nchunk; ch += THREADS) {
          float v[8];
          Elem<T>::load8(xr + ch * 8, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = cta_max<THREADS>(amax, red);
        const RowQuant rq = make_row_quant(amax);
        const float sc = rq.scale;
#pragma unroll
        for (int c = 0; c < kPackChunks; ++c) {
          const int ch = threadIdx.x + c * THREADS;
          if (ch < nchunk) {
            float v[8];
            raw[c].unpack(v);
            const uint2 o = quant8(v, rq);
            for (int k = 0; k < K; ++k)
              if (s_pos[k] >= 0) __stcs(reinterpret_cast<uint2*>(out + static_cast<int64_t>(s_pos[k]) * cols + ch * 8), o);
          }
        }
        for (int ch = threadIdx.x + kPackChunks * THREADS; ch < nchunk; ch += THREADS) {
          float v[8];
          Elem<T>::load8(xr + ch * 8, v);
          const uint2 o = quant8(v, rq);
          for (int k = 0; k < K; ++k)
            if (s_pos[k] >= 0) __stcs(reinterpret_cast<uint2*>(out + static_cast<int64_t>(s_pos[k]) * cols + ch * 8), o);
        }
        for (int k = threadIdx.x; k < K; k += THREADS)
          if (s_pos[k] >= 0) a.send_scales[s_pos[k]] = sc;
      } else {
        // per copy: row * smooth row of its expert (fp32 product), own maximum, own scale
        for (int k = 0; k < K; ++k) {
          const int pos = s_pos[k];                        // uniform over the CTA
          if (pos < 0) continue;
          const float* sm = a.smooth + (a.smooth_rows > 1 ? static_cast<int64_t>(s_key[k]) * cols : 0);
          auto value = [&](int c, int ch, float (&v)[8]) {
            if (c >= 0) raw[c].unpack(v); else Elem<T>::load8(xr + ch * 8, v);
            float m[8];
            Elem<float>::load8(sm + ch * 8, m);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], m[i]);
          };
          float amax = 0.f;
#pragma unroll
          for (int c = 0; c < kPackChunks; ++c) {
            const int ch = threadIdx.x + c * THREADS;
            if (ch < nchunk) {
              float v[8];
              value(c, ch, v);
#pragma unroll
              for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            }
          }
          for (int ch = threadIdx.x + kPackChunks * THREADS; ch < nchunk; ch += THREADS) {
            float v[8];
            value(-1, ch, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
          }
          amax = cta_max<THREADS>(amax, red);
          const RowQuant rq = make_row_quant(amax);
          int8_t* orow = out + static_cast<int64_t>(pos) * cols;
#pragma unroll
          for (int c = 0; c < kPackChunks; ++c) {
            const int ch = threadIdx.x + c * THREADS;
            if (ch < nchunk) {
              float v[8];
              value(c, ch, v);
              __stcs(reinterpret_cast<uint2*>(orow + ch * 8), quant8(v, rq));
            }
          }
          for (int ch = threadIdx.x + kPackChunks * THREADS; ch < nchunk; ch += THREADS) {
            float v[8];
            value(-1, ch, v);
            __stcs(reinterpret_cast<uint2*>(orow + ch * 8), quant8(v, rq));
          }
          if (threadIdx.x == 0) a.send_scales[pos] = rq.scale;
        }
      }
    } else {
      T* out = static_cast<T*>(a.send_rows);
      const int nvec = cols * static_cast<int>(sizeof(T)) / 16;
      const uint4* sp = reinterpret_cast<const uint4*>(xr);
      for (int vi = threadIdx.x; vi < nvec; vi += THREADS) {
        const uint4 val = sp[vi];
        for (int k = 0; k < K; ++k)
          if (s_pos[k] >= 0) reinterpret_cast<uint4*>(out + static_cast<int64_t>(s_pos[k]) * cols)[vi] = val;
      }
      const float pass = a.passthrough_scale ? a.passthrough_scale[t] : 0.f;
      for (int k = threadIdx.x; k < K; k += THREADS)
        if (s_pos[k] >= 0) a.send_scales[s_pos[k]] = pass;
    }
  }
}

template <typename T, bool kSortInside>
static void launch_pack(const void* x, const PackArgs& a, int quant_mode, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const bool small = a.cols / 8 <= 128 * kPackChunks;
  const int grid = grid_for(a.tokens, small ? 10 : 5);
#define TAB_PACK(Q, TH, SM) dispatch_pack_kernel<T, Q, TH, kSortInside, SM><<<grid, TH, 0, st>>>(xp, a)
  if (quant_mode == 2 && a.smooth != nullptr) {
    if (small) TAB_PACK(true, 128, true); else TAB_PACK(true, 256, true);
  } else if (quant_mode == 2) {
    if (small) TAB_PACK(true, 128, false); else TAB_PACK(true, 256, false);
  } else {
    if (small) TAB_PACK(false, 128, false); else TAB_PACK(false, 256, false);
  }
#undef TAB_PACK
}

// ---- receiver side ---------------------------------------------------------------------------------
// plan = wire_off[R*E_l] (index s*E_l+e) ++ exp_off[R*E_l + 1] (index e*R+s, last = total rows).
__global__ void __launch_bounds__(1024) exchange_plan_kernel(const int32_t* __restrict__ recv_counts, int R, int E_l,
                                                            int slot_rows, int nums_type, int32_t* __restrict__ plan,
                                                            int64_t* __restrict__ expert_token_nums,
                                                            int32_t* __restrict__ ep_recv_count) {
  __shared__ int s_wire[kMaxExperts];
  __shared__ int s_exp[kMaxExperts];
  __shared__ int s_warp[33];
  const int n = R * E_l;
  for (int i = threadIdx.x; i < n; i += 1024) {
    const int c = max(recv_counts[i], 0);
    s_wire[i] = c;                       // i = s*E_l + e
    const int s = i / E_l, e = i - s * E_l;
    s_exp[e * R + s] = c;
    ep_recv_count[e * R + s] = c;
  }
  __syncthreads();
  block_exclusive_scan(s_wire, n, s_warp);
  const int total = block_exclusive_scan(s_exp, n, s_warp);
  for (int i = threadIdx.x; i < n; i += 1024) {
    const int s = i / E_l;
    int w = s_wire[i];
    if (slot_rows > 0) w = w - s_wire[s * E_l] + s * slot_rows;  // offset inside the source's fixed slot
    plan[i] = w;
    plan[n + i] = s_exp[i];
  }
  if (threadIdx.x == 0) plan[2 * n] = total;
  for (int e = threadIdx.x; e < E_l; e += 1024) {
    const int begin = s_exp[e * R];
    const int end = (e + 1 < E_l) ? s_exp[(e + 1) * R] : total;
    expert_token_nums[e] = nums_type == 1 ? static_cast<int64_t>(end - begin) : static_cast<int64_t>(end);
  }
}

// Last index b in [lo, hi) with off[b] <= i (off is non-decreasing on the range, off[lo] <= i).
__device__ __forceinline__ int last_le(const int32_t* __restrict__ off, int lo, int hi, int i) {
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (off[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kRowCopyThreads) exchange_rows_kernel(const uint4* __restrict__ src, const float* __restrict__ src_scales,
                                                            const int32_t* __restrict__ plan, int R, int E_l,
                                                            int slot_rows, int direction, int vec_per_row,
                                                            int64_t dst_rows, int zero_fill, uint4* __restrict__ dst,
                                                            float* __restrict__ dst_scales) {
  const int n = R * E_l;
  const int32_t* wire_off = plan;
  const int32_t* exp_off = plan + n;
  const int total = exp_off[n];
  for (int64_t i = blockIdx.x; i < dst_rows; i += gridDim.x) {
    int64_t srow = -1;
    if (direction == 0) {           // dst in expert order
      if (i < total) {
        const int b = last_le(exp_off, 0, n, static_cast<int>(i));   // b = e*R + s
        const int e = b / R, s = b - e * R;
        srow = wire_off[s * E_l + e] + (i - exp_off[b]);
      }
    } else {                        // dst is the wire buffer
      int lo = 0, hi = n;
      bool in_range = true;
      if (slot_rows > 0) {
        const int s = static_cast<int>(i / slot_rows);
        in_range = s < R;
        lo = s * E_l;
        hi = lo + E_l;
      } else {
        in_range = i < total;
      }
      if (in_range) {
        const int b = last_le(wire_off, lo, hi, static_cast<int>(i));  // b = s*E_l + e
        const int s = b / E_l, e = b - s * E_l;
        const int eb = e * R + s;
        const int64_t j = i - wire_off[b];
        if (j < exp_off[eb + 1] - exp_off[eb]) srow = exp_off[eb] + j;
      }
    }
    uint4* dp = dst + i * vec_per_row;
    if (srow >= 0) {
      copy_row16<kRowCopyThreads>(dp, src + srow * vec_per_row, vec_per_row);
      if (dst_scales && threadIdx.x == 0) dst_scales[i] = src_scales[srow];
    } else if (zero_fill) {
      for (int v = threadIdx.x; v < vec_per_row; v += kRowCopyThreads) dp[v] = make_uint4(0, 0, 0, 0);
      if (dst_scales && threadIdx.x == 0) dst_scales[i] = 0.f;
    }
  }
}

// Optional inputs of the combine (all may be absent): a token mask, and the special experts of the second-generation
// operator -- pairs whose expert id is >= num_experts stand for rows that are formed here instead of being gathered:
// zero experts (0), copy experts (the token itself, ori_x) and constant experts (alpha_1[c] * ori_x + alpha_2[c] * v[c]).
struct CombineExtra {
  const uint8_t* mask;         // [T] or null: a 0 byte gives an all-zero output row
  const int32_t* expert_ids;   // [T, K], read only when special experts exist
  int num_experts, zero_num, copy_num, const_num;
  const void* ori_x;           // [T, H]
  const void* alpha_1;         // [const_num, H]
  const void* alpha_2;         // [const_num, H]
  const void* const_v;         // [const_num, H]
  // expert-parallel combine over peer memory: once every CTA has read its rows, the last one tells the ack_ranks peers
  // (flag slots ack_peer_flags[r], next sequence number from ack_sig_counter) that their return buffers may be reused
  unsigned long long* const* ack_peer_flags;
  unsigned long long* ack_sig_counter;
  unsigned int* done_counter;
  int ack_ranks;
};

// out[t] = sum_k w[t,k] * rows[idx[t*K+k]] (+ shared[t]); fp32, separate multiply and add, ascending k.  A negative
// index (a pair that was dropped and is no special expert) contributes 0.
// The bandwidth-bound case on its own: many tokens, no mask, no special experts, nothing to acknowledge.  A token with a
// pair that has no row (negative index) is left to combine_kernel, launched after this one for those tokens only.
template <typename T>
__global__ void __launch_bounds__(256) combine_plain_kernel(const T* __restrict__ rows, const int32_t* __restrict__ expand_idx,
                                                            const float* __restrict__ weights, const T* __restrict__ shared,
                                                            int64_t tokens, int K, int cols, T* __restrict__ out) {
  extern __shared__ int s_meta[];  // [K] positions, [K] weights
  int* s_pos = s_meta;
  float* s_w = reinterpret_cast<float*>(s_meta + K);
  const int nchunk = cols >> 3;
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    __syncthreads();
    int no_row = 0;
    for (int k = threadIdx.x; k < K; k += 256) {
      const int pos = expand_idx[t * K + k];
      no_row |= pos < 0 ? 1 : 0;
      s_pos[k] = pos;
      s_w[k] = weights[t * K + k];
    }
    if (__syncthreads_or(no_row)) continue;
    for (int ch = threadIdx.x; ch < nchunk; ch += 256) {
      float acc[8];
#pragma unroll 4
      for (int k = 0; k < K; ++k) {
        float v[8];
        Elem<T>::load8(rows + static_cast<int64_t>(s_pos[k]) * cols + ch * 8, v);
        const float w = s_w[k];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float term = __fmul_rn(w, v[i]);
          acc[i] = k == 0 ? term : __fadd_rn(acc[i], term);
        }
      }
      if (shared) {
        float v[8];
        Elem<T>::load8(shared + t * cols + ch * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
      }
      Elem<T>::store8(out + t * cols + ch * 8, acc);
    }
  }
}

// Second pass after combine_plain_kernel: the tokens it skipped (a pair without a row).  Every thread looks at one token
// of a block of 256; the flagged ones, normally none, are then summed by the whole CTA with an exact zero in place of the
// missing rows.  A few CTAs read T*K indices: the pass costs little more than its launch.
template <typename T>
__global__ void __launch_bounds__(256) combine_fixup_kernel(const T* __restrict__ rows, const int32_t* __restrict__ expand_idx,
                                                            const float* __restrict__ weights, const T* __restrict__ shared,
                                                            int64_t tokens, int K, int cols, T* __restrict__ out) {
  __shared__ int s_list[256];
  __shared__ int s_count;
  const int nchunk = cols >> 3;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * 256; base < tokens; base += static_cast<int64_t>(gridDim.x) * 256) {
    __syncthreads();
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    const int64_t mine = base + threadIdx.x;
    if (mine < tokens) {
      bool no_row = false;
      for (int k = 0; k < K; ++k) no_row |= expand_idx[mine * K + k] < 0;
      if (no_row) s_list[atomicAdd(&s_count, 1)] = threadIdx.x;
    }
    __syncthreads();
    const int n = s_count;
    for (int q = 0; q < n; ++q) {
      const int64_t t = base + s_list[q];
      for (int ch = threadIdx.x; ch < nchunk; ch += 256) {
        float acc[8];
        for (int k = 0; k < K; ++k) {
          const int pos = expand_idx[t * K + k];
          float v[8];
          Elem<T>::load8(rows + static_cast<int64_t>(pos < 0 ? 0 : pos) * cols + ch * 8, v);
          const float w = weights[t * K + k];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float term = __fmul_rn(w, pos < 0 ? 0.f : v[i]);
            acc[i] = k == 0 ? term : __fadd_rn(acc[i], term);
          }
        }
        if (shared) {
          float v[8];
          Elem<T>::load8(shared + t * cols + ch * 8, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
        }
        Elem<T>::store8(out + t * cols + ch * 8, acc);
      }
    }
  }
}

template <typename T, bool kExtra, bool kSliced>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ rows, const int32_t* __restrict__ expand_idx,
                                                      const float* __restrict__ weights, const T* __restrict__ shared,
                                                      int64_t tokens, int K, int cols, int slices, T* __restrict__ out,
                                                      const CombineExtra ex) {
  extern __shared__ int s_meta[];  // [K] positions, [K] weights, [K] special kinds
  int* s_pos = s_meta;
  float* s_w = reinterpret_cast<float*>(s_meta + K);
  int* s_kind = s_meta + 2 * K;    // -1: gathered row; else index among the special experts
  const int nchunk_all = cols >> 3;
  const int per_slice = kSliced ? (nchunk_all + slices - 1) / slices : nchunk_all;
  const int specials = kExtra ? ex.zero_num + ex.copy_num + ex.const_num : 0;
  // work item = (token, column slice): with few tokens (kSliced) a row is cut into slices so that the launch still fills
  // the GPU; otherwise an item is a whole token and the column loop has fixed bounds
  for (int64_t item = blockIdx.x; item < (kSliced ? tokens * slices : tokens); item += gridDim.x) {
    const int64_t t = kSliced ? item / slices : item;
    const int ch0 = kSliced ? static_cast<int>(item - t * slices) * per_slice : 0;
    const int nchunk = kSliced ? min(ch0 + per_slice, nchunk_all) : nchunk_all;
    if (kExtra && ex.mask != nullptr && ex.mask[t] == 0) {     // uniform over the CTA
      for (int ch = ch0 + threadIdx.x; ch < nchunk; ch += 256) *reinterpret_cast<uint4*>(out + t * cols + ch * 8) = make_uint4(0, 0, 0, 0);
      continue;
    }
    __syncthreads();
    int no_row = 0;
    for (int k = threadIdx.x; k < K; k += 256) {
      const int pos = expand_idx[t * K + k];
      no_row |= pos < 0 ? 1 : 0;
      s_pos[k] = pos;
      s_w[k] = weights[t * K + k];
      if constexpr (kExtra) {
        const int id = specials > 0 ? ex.expert_ids[t * K + k] : 0;
        s_kind[k] = (specials > 0 && id >= ex.num_experts && id < ex.num_experts + specials) ? id - ex.num_experts : -1;
      }
    }
    no_row = __syncthreads_or(no_row);
    if (!kExtra && !no_row) {
      // every pair of this token has a row (the common case): K plain gathers per chunk, nothing to select
      for (int ch = ch0 + threadIdx.x; ch < nchunk; ch += 256) {
        float acc[8];
#pragma unroll 4
        for (int k = 0; k < K; ++k) {
          float v[8];
          Elem<T>::load8(rows + static_cast<int64_t>(s_pos[k]) * cols + ch * 8, v);
          const float w = s_w[k];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float term = __fmul_rn(w, v[i]);
            acc[i] = k == 0 ? term : __fadd_rn(acc[i], term);
          }
        }
        if (shared) {
          float v[8];
          Elem<T>::load8(shared + t * cols + ch * 8, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
        }
        Elem<T>::store8(out + t * cols + ch * 8, acc);
      }
      continue;
    }
    for (int ch = ch0 + threadIdx.x; ch < nchunk; ch += 256) {
      float acc[8];
#pragma unroll 4
      for (int k = 0; k < K; ++k) {
        float v[8];
        const int kind = kExtra ? s_kind[k] : -1;
        if (kind < 0) {
          // the load is unconditional (row 0 stands in for a pair that has no row) so that the K loads of a chunk are in
          // flight together; a select then puts the exact zero of a dropped pair in place
          const int pos = s_pos[k];
          Elem<T>::load8(rows + static_cast<int64_t>(pos < 0 ? 0 : pos) * cols + ch * 8, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = pos < 0 ? 0.f : v[i];
        } else if (kind < ex.zero_num) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = 0.f;
        } else {
          Elem<T>::load8(static_cast<const T*>(ex.ori_x) + t * cols + ch * 8, v);
          if (kind >= ex.zero_num + ex.copy_num) {
            const int64_t c = kind - ex.zero_num - ex.copy_num;
            float a1[8], a2[8], cv[8];
            Elem<T>::load8(static_cast<const T*>(ex.alpha_1) + c * cols + ch * 8, a1);
            Elem<T>::load8(static_cast<const T*>(ex.alpha_2) + c * cols + ch * 8, a2);
            Elem<T>::load8(static_cast<const T*>(ex.const_v) + c * cols + ch * 8, cv);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(__fmul_rn(a1[i], v[i]), __fmul_rn(a2[i], cv[i]));
          }
        }
        const float w = s_w[k];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float term = __fmul_rn(w, v[i]);
          acc[i] = k == 0 ? term : __fadd_rn(acc[i], term);
        }
      }
      if (shared) {
        float v[8];
        Elem<T>::load8(shared + t * cols + ch * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
      }
      Elem<T>::store8(out + t * cols + ch * 8, acc);
    }
  }
  if (ex.ack_peer_flags != nullptr) {
    __shared__ int s_last;
    __syncthreads();                       // every thread's loads of the returned rows have been consumed
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = atomicInc(ex.done_counter, gridDim.x - 1) == gridDim.x - 1 ? 1 : 0;   // wraps to 0 for the next launch
    }
    __syncthreads();
    if (s_last) {
      const unsigned long long v = *ex.ack_sig_counter + 1;
      __syncthreads();
      if (threadIdx.x < ex.ack_ranks)
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(ex.ack_peer_flags[threadIdx.x]), "l"(v) : "memory");
      if (threadIdx.x == 0) *ex.ack_sig_counter = v;
    }
  }
}

static int elem_size(int dtype) {
  switch (dtype) {
    case TAB_BF16: case TAB_F16: return 2;
    case TAB_F32: case TAB_I32: return 4;
    case TAB_I8: return 1;
    default: return 0;
  }
}

}  // namespace tab

using namespace tab;

extern "C" int tab_moe_init_routing_workspace_bytes(int64_t T, int64_t K, int64_t expert_bound, size_t* bytes) {
  if (!bytes || T < 0 || K <= 0 || expert_bound <= 0 || expert_bound > kMaxExperts)
    return fail(TAB_ERR_BAD_ARG, "init_routing: T=%lld K=%lld expert_bound=%lld (bound must be in [1, %d])", (long long)T, (long long)K, (long long)expert_bound, kMaxExperts);
  *bytes = sort_scratch_bytes(T * K, expert_bound + 1, false);
  return TAB_OK;
}

extern "C" int tab_moe_init_routing(const void* x, int x_dtype, const int32_t* row_idx, const int32_t* expert_idx,
                                    int64_t T, int64_t K, int64_t H, int64_t active_num, int64_t expert_bound,
                                    void* expanded_x, int32_t* expanded_row_idx, int32_t* expanded_expert_idx,
                                    void* workspace, size_t workspace_bytes, tab_stream_t stream) {
  size_t need = 0;
  int rc = tab_moe_init_routing_workspace_bytes(T, K, expert_bound, &need);
  if (rc != TAB_OK) return rc;
  const int es = elem_size(x_dtype);
  if (es != 2 && es != 4) return fail(TAB_ERR_UNSUPPORTED, "init_routing: x dtype %d (want 5, 6 or 15)", x_dtype);
  if (H <= 0 || active_num < 0) return fail(TAB_ERR_BAD_ARG, "init_routing: H=%lld active_num=%lld", (long long)H, (long long)active_num);
  const int64_t n = T * K;
  if (n == 0) return TAB_OK;
  if (n > (1LL << 30)) return fail(TAB_ERR_UNSUPPORTED, "init_routing: T*K too large");
  if (!x || !row_idx || !expert_idx || !expanded_x || !expanded_row_idx || !expanded_expert_idx || !workspace)
    return fail(TAB_ERR_BAD_ARG, "init_routing: null pointer");
  if (workspace_bytes < need) return fail(TAB_ERR_WORKSPACE, "init_routing: workspace %zu < %zu bytes", workspace_bytes, need);
  if ((H * es) % 16 != 0 || !aligned16(x) || !aligned16(expanded_x) || !aligned16(workspace))
    return fail(TAB_ERR_ALIGNMENT, "init_routing: rows must be 16-byte multiples and pointers 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  SortScratch s = carve(workspace, n, expert_bound + 1, false);
  const PairFilter pf = {nullptr, (int)K, 0, (int)expert_bound, 0};
  rc = run_sort(expert_idx, row_idx, n, pf, s, expanded_expert_idx, expanded_row_idx, nullptr, st);
  if (rc != TAB_OK) return rc;
  const int64_t out_rows = (T < active_num ? T : active_num) * K;
  if (out_rows > 0) {
    const int64_t row_bytes = H * es;
    const size_t ring_bytes = static_cast<size_t>(row_bytes) * kBulkStages;
    if (row_bytes >= 512 && ring_bytes <= 192 * 1024 && T >= 32 &&
        cudaFuncSetAttribute(scatter_rows_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ring_bytes)) == cudaSuccess) {
      size_t per_sm = (200 * 1024) / (ring_bytes + 1024);
      if (per_sm > 8) per_sm = 8;
      if (per_sm < 1) per_sm = 1;
      scatter_rows_bulk_kernel<<<grid_for(T, static_cast<int>(per_sm)), 32, ring_bytes, st>>>(
          static_cast<const uint8_t*>(x), expanded_row_idx, T, (int)K, out_rows, static_cast<uint32_t>(row_bytes),
          static_cast<uint8_t*>(expanded_x));
    } else {
      gather_rows_kernel<<<grid_for(out_rows, 16), kRowCopyThreads, 0, st>>>(static_cast<const uint4*>(x), s.sorted_src, (int)T, out_rows,
                                                                (int)(H * es / 16), static_cast<uint4*>(expanded_x));
    }
    rc = check_launch("init_routing gather");
  }
  return rc;
}

extern "C" int tab_moe_dispatch_pack_workspace_bytes(int64_t T, int64_t K, int64_t num_experts, size_t* bytes) {
  if (!bytes || T < 0 || K <= 0 || num_experts <= 0 || num_experts > kMaxExperts)
    return fail(TAB_ERR_BAD_ARG, "dispatch_pack: T=%lld K=%lld experts=%lld (experts must be in [1, %d])", (long long)T, (long long)K, (long long)num_experts, kMaxExperts);
  *bytes = sort_scratch_bytes(T * K, num_experts + 1, true);
  return TAB_OK;
}

extern "C" int tab_moe_dispatch_pack_ex(const void* x, int x_dtype, const int32_t* expert_ids, int64_t T, int64_t K, int64_t H,
                                        int64_t expert_lo, int64_t expert_hi, int drop_outside, const uint8_t* x_active_mask,
                                        const float* smooth, int64_t smooth_rows, const float* passthrough_scale, int64_t pos_limit,
                                        int quant_mode, void* send_rows, float* send_scales, int32_t* expand_idx,
                                        int32_t* expert_counts, int64_t* expert_token_nums, int nums_type, void* workspace,
                                        size_t workspace_bytes, tab_stream_t stream) {
  const int64_t num_experts = expert_hi - expert_lo;
  if (expert_lo < 0 || num_experts <= 0) return fail(TAB_ERR_BAD_ARG, "dispatch_pack: expert range [%lld, %lld)", (long long)expert_lo, (long long)expert_hi);
  size_t need = 0;
  int rc = tab_moe_dispatch_pack_workspace_bytes(T, K, num_experts, &need);
  if (rc != TAB_OK) return rc;
  if (quant_mode != 0 && quant_mode != 2) return fail(TAB_ERR_UNSUPPORTED, "dispatch_pack: quant_mode %d (want 0 or 2)", quant_mode);
  if (x_dtype != TAB_BF16 && x_dtype != TAB_F16) return fail(TAB_ERR_UNSUPPORTED, "dispatch_pack: x dtype %d (want 5 or 15)", x_dtype);
  if (!expert_counts) return fail(TAB_ERR_BAD_ARG, "dispatch_pack: null pointer");
  if (nums_type != 0 && nums_type != 1) return fail(TAB_ERR_BAD_ARG, "dispatch_pack: nums_type %d", nums_type);
  if (smooth && (quant_mode != 2 || (smooth_rows != 1 && smooth_rows != num_experts) || !aligned16(smooth)))
    return fail(TAB_ERR_BAD_ARG, "dispatch_pack: smooth scales need quant_mode 2, 1 or %lld rows (got %lld) and 16-byte alignment", (long long)num_experts, (long long)smooth_rows);
  if (passthrough_scale && quant_mode != 0) return fail(TAB_ERR_BAD_ARG, "dispatch_pack: a pass-through scale needs quant_mode 0");
  cudaStream_t st = as_stream(stream);
  const int64_t n = T * K;
  if (n == 0) {
    cudaError_t e = cudaMemsetAsync(expert_counts, 0, num_experts * sizeof(int32_t), st);
    if (e == cudaSuccess && expert_token_nums) e = cudaMemsetAsync(expert_token_nums, 0, num_experts * sizeof(int64_t), st);
    return e == cudaSuccess ? TAB_OK : fail(TAB_ERR_CUDA, "dispatch_pack: memset: %s", cudaGetErrorString(e));
  }
  if (n > (1LL << 30) || K > 256) return fail(TAB_ERR_UNSUPPORTED, "dispatch_pack: T*K too large or K > 256");
  if (!x || !expert_ids || !send_rows || !send_scales || !expand_idx || !workspace)
    return fail(TAB_ERR_BAD_ARG, "dispatch_pack: null pointer");
  if (workspace_bytes < need) return fail(TAB_ERR_WORKSPACE, "dispatch_pack: workspace %zu < %zu bytes", workspace_bytes, need);
  if (H <= 0 || H % 16 != 0 || !aligned16(x) || !aligned16(send_rows) || !aligned16(workspace))
    return fail(TAB_ERR_ALIGNMENT, "dispatch_pack: H=%lld must be a multiple of 16 and pointers 16-byte aligned", (long long)H);
  SortScratch s = carve(workspace, n, num_experts + 1, true);
  PackArgs a = {};
  a.expand_idx = expand_idx;
  a.tokens = T; a.K = (int)K; a.cols = (int)H;
  a.send_rows = send_rows; a.send_scales = send_scales;
  a.counts = expert_counts; a.nums64 = expert_token_nums;
  a.num_experts = (int)num_experts; a.nums_type = nums_type;
  a.expert_ids = expert_ids;
  a.sorted_src = s.sorted_src;
  a.smooth = smooth; a.smooth_rows = (int)smooth_rows;
  a.passthrough_scale = passthrough_scale;
  a.pos_limit = pos_limit > 0 && pos_limit < 0x7fffffffLL ? (int)pos_limit : 0x7fffffff;
  a.pf = PairFilter{x_active_mask, (int)K, (int)expert_lo, (int)expert_hi, drop_outside};
  if (n <= kSmallPairs) {
    // decode-sized batches: the sort runs inside the pack kernel, one launch in all
    if (x_dtype == TAB_BF16) launch_pack<__nv_bfloat16, true>(x, a, quant_mode, st);
    else launch_pack<__half, true>(x, a, quant_mode, st);
    return check_launch("dispatch_pack");
  }
  rc = run_sort(expert_ids, nullptr, n, a.pf, s, s.sorted_expert, expand_idx, expert_counts, st);
  if (rc != TAB_OK) return rc;
  if (x_dtype == TAB_BF16) launch_pack<__nv_bfloat16, false>(x, a, quant_mode, st);
  else launch_pack<__half, false>(x, a, quant_mode, st);
  return check_launch("dispatch_pack");
}

extern "C" int tab_moe_dispatch_pack(const void* x, int x_dtype, const int32_t* expert_ids, int64_t T, int64_t K,
                                     int64_t H, int64_t num_experts, int quant_mode, void* send_rows,
                                     float* send_scales, int32_t* expand_idx, int32_t* expert_counts,
                                     int64_t* expert_token_nums, int nums_type, void* workspace, size_t workspace_bytes,
                                     tab_stream_t stream) {
  return tab_moe_dispatch_pack_ex(x, x_dtype, expert_ids, T, K, H, 0, num_experts, 0, nullptr, nullptr, 0, nullptr, 0, quant_mode,
                                  send_rows, send_scales, expand_idx, expert_counts, expert_token_nums, nums_type, workspace,
                                  workspace_bytes, stream);
}

extern "C" int tab_moe_exchange_plan(const int32_t* recv_counts, int64_t R, int64_t E_l, int64_t slot_rows,
                                     int nums_type, int32_t* plan, int64_t* expert_token_nums,
                                     int32_t* ep_recv_count, tab_stream_t stream) {
  if (!recv_counts || !plan || !expert_token_nums || !ep_recv_count) return fail(TAB_ERR_BAD_ARG, "exchange_plan: null pointer");
  if (R <= 0 || E_l <= 0 || R * E_l > kMaxExperts || slot_rows < 0 || slot_rows > (1LL << 30))
    return fail(TAB_ERR_BAD_ARG, "exchange_plan: R=%lld E_l=%lld (R*E_l must be in [1, %d])", (long long)R, (long long)E_l, kMaxExperts);
  if (nums_type != 0 && nums_type != 1) return fail(TAB_ERR_BAD_ARG, "exchange_plan: nums_type %d", nums_type);
  exchange_plan_kernel<<<1, 1024, 0, as_stream(stream)>>>(recv_counts, (int)R, (int)E_l, (int)slot_rows, nums_type, plan,
                                                         expert_token_nums, ep_recv_count);
  return check_launch("exchange_plan");
}

extern "C" int tab_moe_exchange_rows(const void* src, const float* src_scales, const int32_t* plan, int64_t R,
                                     int64_t E_l, int64_t slot_rows, int direction, int64_t row_bytes,
                                     int64_t dst_rows, int zero_fill, void* dst, float* dst_scales,
                                     tab_stream_t stream) {
  if (dst_rows == 0) return TAB_OK;
  if (!src || !plan || !dst) return fail(TAB_ERR_BAD_ARG, "exchange_rows: null pointer");
  if (R <= 0 || E_l <= 0 || R * E_l > kMaxExperts || dst_rows < 0 || dst_rows > (1LL << 30) || (direction != 0 && direction != 1))
    return fail(TAB_ERR_BAD_ARG, "exchange_rows: bad R/E_l/rows/direction");
  if ((dst_scales != nullptr) != (src_scales != nullptr)) return fail(TAB_ERR_BAD_ARG, "exchange_rows: scales must be given on both sides or neither");
  if (row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(src) || !aligned16(dst))
    return fail(TAB_ERR_ALIGNMENT, "exchange_rows: row_bytes=%lld must be a multiple of 16 and pointers 16-byte aligned", (long long)row_bytes);
  exchange_rows_kernel<<<grid_for(dst_rows, 16), kRowCopyThreads, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(src), src_scales, plan, (int)R, (int)E_l, (int)slot_rows, direction, (int)(row_bytes / 16),
      dst_rows, zero_fill, static_cast<uint4*>(dst), dst_scales);
  return check_launch("exchange_rows");
}

static int combine_impl(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                        const void* shared, int64_t T, int64_t K, int64_t H, void* out, const uint8_t* x_active_mask,
                        const int32_t* expert_ids, int64_t num_experts, int64_t zero_expert_num, int64_t copy_expert_num,
                        int64_t const_expert_num, const void* ori_x, const void* const_expert_alpha_1,
                        const void* const_expert_alpha_2, const void* const_expert_v, void* const* ack_peer_flags,
                        void* ack_sig_counter, void* done_counter, int64_t ack_ranks, tab_stream_t stream) {
  if (ack_peer_flags != nullptr && (T <= 0 || !ack_sig_counter || !done_counter || ack_ranks < 1 || ack_ranks > 256))
    return fail(TAB_ERR_BAD_ARG, "combine: the acknowledgement needs T > 0, both counters and 1..256 ranks");
  if (T < 0 || K <= 0 || K > 1024 || H <= 0) return fail(TAB_ERR_BAD_ARG, "combine: T=%lld K=%lld H=%lld", (long long)T, (long long)K, (long long)H);
  if (T == 0) return TAB_OK;
  if (!rows || !expand_idx || !expert_scales || !out) return fail(TAB_ERR_BAD_ARG, "combine: null pointer");
  if (H % 8 != 0 || !aligned16(rows) || !aligned16(out) || (shared && !aligned16(shared)))
    return fail(TAB_ERR_ALIGNMENT, "combine: H=%lld must be a multiple of 8 and pointers 16-byte aligned", (long long)H);
  if (zero_expert_num < 0 || copy_expert_num < 0 || const_expert_num < 0) return fail(TAB_ERR_BAD_ARG, "combine: negative special expert count");
  const int64_t specials = zero_expert_num + copy_expert_num + const_expert_num;
  if (specials > 0 && (!expert_ids || num_experts <= 0)) return fail(TAB_ERR_BAD_ARG, "combine: special experts need expert_ids and the number of routed experts");
  if (copy_expert_num + const_expert_num > 0 && (!ori_x || !aligned16(ori_x))) return fail(TAB_ERR_BAD_ARG, "combine: copy and constant experts need ori_x (16-byte aligned)");
  if (const_expert_num > 0 && (!const_expert_alpha_1 || !const_expert_alpha_2 || !const_expert_v || !aligned16(const_expert_alpha_1) ||
                               !aligned16(const_expert_alpha_2) || !aligned16(const_expert_v)))
    return fail(TAB_ERR_BAD_ARG, "combine: constant experts need alpha_1, alpha_2 and v (16-byte aligned)");
  cudaStream_t st = as_stream(stream);
  // few tokens: cut every row into slices of at least 128 16-byte chunks until the launch has about four CTAs per SM
  int slices = 1;
  while (T * slices < 4 * kNumSMs && (H / 8) / (slices * 2) >= 128) slices *= 2;
  const int grid = grid_for(T * slices, 8);
  const size_t smem = static_cast<size_t>(K) * 12;
  const bool extra = x_active_mask != nullptr || specials > 0;
  const CombineExtra ex = {x_active_mask, expert_ids, (int)num_experts, (int)zero_expert_num, (int)copy_expert_num, (int)const_expert_num,
                           ori_x, const_expert_alpha_1, const_expert_alpha_2, const_expert_v,
                           reinterpret_cast<unsigned long long* const*>(ack_peer_flags), static_cast<unsigned long long*>(ack_sig_counter),
                           static_cast<unsigned int*>(done_counter), (int)ack_ranks};
  // many tokens and none of the optional inputs: the lean kernel, then a small pass for the tokens it left (if any)
  if (!extra && ack_peer_flags == nullptr && slices == 1 && T >= 2048) {
    const int fix_grid = static_cast<int>((T + 255) / 256 < 2 * kNumSMs ? (T + 255) / 256 : 2 * kNumSMs);
    const size_t smem2 = static_cast<size_t>(K) * 8;
    if (dtype == TAB_BF16) {
      const __nv_bfloat16* r = static_cast<const __nv_bfloat16*>(rows);
      const __nv_bfloat16* sh = static_cast<const __nv_bfloat16*>(shared);
      combine_plain_kernel<__nv_bfloat16><<<grid, 256, smem2, st>>>(r, expand_idx, expert_scales, sh, T, (int)K, (int)H, static_cast<__nv_bfloat16*>(out));
      combine_fixup_kernel<__nv_bfloat16><<<fix_grid, 256, 0, st>>>(r, expand_idx, expert_scales, sh, T, (int)K, (int)H, static_cast<__nv_bfloat16*>(out));
    } else if (dtype == TAB_F16) {
      const __half* r = static_cast<const __half*>(rows);
      const __half* sh = static_cast<const __half*>(shared);
      combine_plain_kernel<__half><<<grid, 256, smem2, st>>>(r, expand_idx, expert_scales, sh, T, (int)K, (int)H, static_cast<__half*>(out));
      combine_fixup_kernel<__half><<<fix_grid, 256, 0, st>>>(r, expand_idx, expert_scales, sh, T, (int)K, (int)H, static_cast<__half*>(out));
    } else {
      return fail(TAB_ERR_UNSUPPORTED, "combine: dtype %d (want 5 or 15)", dtype);
    }
    return check_launch("combine", 2);
  }
#define TAB_COMBINE(TYPE, EX, SL)                                                                                               \
  combine_kernel<TYPE, EX, SL><<<grid, 256, smem, st>>>(static_cast<const TYPE*>(rows), expand_idx, expert_scales,              \
                                                        static_cast<const TYPE*>(shared), T, (int)K, (int)H, slices,           \
                                                        static_cast<TYPE*>(out), ex)
#define TAB_COMBINE2(TYPE, EX)                                                                                                  \
  do { if (slices > 1) TAB_COMBINE(TYPE, EX, true); else TAB_COMBINE(TYPE, EX, false); } while (0)
  if (dtype == TAB_BF16) {
    if (extra) TAB_COMBINE2(__nv_bfloat16, true); else TAB_COMBINE2(__nv_bfloat16, false);
  } else if (dtype == TAB_F16) {
    if (extra) TAB_COMBINE2(__half, true); else TAB_COMBINE2(__half, false);
  } else {
    return fail(TAB_ERR_UNSUPPORTED, "combine: dtype %d (want 5 or 15)", dtype);
  }
#undef TAB_COMBINE2
#undef TAB_COMBINE
  return check_launch("combine");
}

extern "C" int tab_moe_combine_ex(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                                  const void* shared, int64_t T, int64_t K, int64_t H, void* out, const uint8_t* x_active_mask,
                                  const int32_t* expert_ids, int64_t num_experts, int64_t zero_expert_num, int64_t copy_expert_num,
                                  int64_t const_expert_num, const void* ori_x, const void* const_expert_alpha_1,
                                  const void* const_expert_alpha_2, const void* const_expert_v, tab_stream_t stream) {
  return combine_impl(rows, dtype, expand_idx, expert_scales, shared, T, K, H, out, x_active_mask, expert_ids, num_experts, zero_expert_num,
                      copy_expert_num, const_expert_num, ori_x, const_expert_alpha_1, const_expert_alpha_2, const_expert_v, nullptr,
                      nullptr, nullptr, 0, stream);
}

extern "C" int tab_moe_combine_ack(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                                   const void* shared, int64_t T, int64_t K, int64_t H, void* out, const uint8_t* x_active_mask,
                                   const int32_t* expert_ids, int64_t num_experts, int64_t zero_expert_num, int64_t copy_expert_num,
                                   int64_t const_expert_num, const void* ori_x, const void* const_expert_alpha_1,
                                   const void* const_expert_alpha_2, const void* const_expert_v, void* const* ack_peer_flags,
                                   void* ack_sig_counter, void* done_counter, int64_t ack_ranks, tab_stream_t stream) {
  if (!ack_peer_flags) return fail(TAB_ERR_BAD_ARG, "combine_ack: null flag table");
  return combine_impl(rows, dtype, expand_idx, expert_scales, shared, T, K, H, out, x_active_mask, expert_ids, num_experts, zero_expert_num,
                      copy_expert_num, const_expert_num, ori_x, const_expert_alpha_1, const_expert_alpha_2, const_expert_v,
                      ack_peer_flags, ack_sig_counter, done_counter, ack_ranks, stream);
}

extern "C" int tab_moe_combine(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                               const void* shared, int64_t T, int64_t K, int64_t H, void* out, tab_stream_t stream) {
  return tab_moe_combine_ex(rows, dtype, expand_idx, expert_scales, shared, T, K, H, out, nullptr, nullptr, 0, 0, 0, 0, nullptr,
                            nullptr, nullptr, nullptr, stream);
}

extern "C" int tab_routing_status(int* status_host, tab_stream_t stream) {
  if (!status_host) return fail(TAB_ERR_BAD_ARG, "routing_status: null pointer");
  cudaStream_t st = as_stream(stream);
  cudaError_t e = cudaStreamSynchronize(st);
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(status_host, g_routing_status, sizeof(int));
  if (e == cudaSuccess && *status_host != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_routing_status, &zero, sizeof(int));
  }
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "routing_status: %s", cudaGetErrorString(e));
  if (*status_host != 0)
    return fail(TAB_ERR_BAD_ARG, "routing: %s%s%s since the last check (clamped / skipped, nothing was accessed out of range)",
                (*status_host & 1) ? "an expert id outside [0, bound)" : "", (*status_host & 3) == 3 ? " and " : "",
                (*status_host & 2) ? "a row_idx value outside [0, T*K)" : "");
  return TAB_OK;
}

// ---- routing without caller-provided scratch -----------------------------------------------------------
// Same work as tab_moe_init_routing, but the sort's scratch (chunk histograms, expert totals, sorted source
// rows) lives in a fixed array inside the library's device image instead of a caller-supplied workspace.
namespace tab {

constexpr int64_t kStaticMaxPairs = 32768;    // T*K
constexpr int64_t kStaticMaxExperts = 512;    // expert_bound
constexpr size_t kStaticScratchBytes = 256 * 1024;
static_assert(((kStaticMaxPairs / kChunk) * (kStaticMaxExperts + 1) + (kStaticMaxExperts + 1) + 4 + kStaticMaxPairs) * 4 + 256 <=
                  kStaticScratchBytes, "static routing scratch must hold the largest accepted problem");

// One copy per GPU that loads the library, resident until the process exits.
static __device__ __align__(256) unsigned char g_static_routing_scratch[kStaticScratchBytes];

static std::mutex g_static_mutex;
static void* g_static_scratch_addr[64] = {nullptr};

// In host code `g_static_routing_scratch` is only a handle for the symbol, not a device address; the address on
// the current device comes from cudaGetSymbolAddress, looked up once per device and remembered.
static int static_scratch_on_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "init_routing_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(TAB_ERR_UNSUPPORTED, "init_routing_static: device index %d", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_routing_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(TAB_ERR_CUDA, "init_routing_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return TAB_OK;
}

}  // namespace tab

extern "C" int tab_moe_init_routing_static(const void* x, int x_dtype, const int32_t* row_idx, const int32_t* expert_idx,
                                           int64_t T, int64_t K, int64_t H, int64_t active_num, int64_t expert_bound,
                                           void* expanded_x, int32_t* expanded_row_idx, int32_t* expanded_expert_idx,
                                           tab_stream_t stream) {
  if (T < 0 || K <= 0 || expert_bound <= 0)
    return fail(TAB_ERR_BAD_ARG, "init_routing_static: T=%lld K=%lld expert_bound=%lld", (long long)T, (long long)K, (long long)expert_bound);
  if (T > kStaticMaxPairs / K || T * K > kStaticMaxPairs || expert_bound > kStaticMaxExperts)
    return fail(TAB_ERR_UNSUPPORTED,
                "init_routing_static: T*K=%lld (max %lld) or expert_bound=%lld (max %lld) exceeds the built-in scratch; "
                "use tab_moe_init_routing with a workspace",
                (long long)(T * K), (long long)kStaticMaxPairs, (long long)expert_bound, (long long)kStaticMaxExperts);
  if (T * K == 0) return TAB_OK;
  void* scratch = nullptr;
  int rc = static_scratch_on_current_device(&scratch);
  if (rc != TAB_OK) return rc;
  // Every scratch word the kernels read is written earlier in the same call (histograms, totals and sorted rows
  // are fully overwritten), so nothing left over from the previous call needs clearing.
  return tab_moe_init_routing(x, x_dtype, row_idx, expert_idx, T, K, H, active_num, expert_bound, expanded_x,
                              expanded_row_idx, expanded_expert_idx, scratch, kStaticScratchBytes, stream);
}

// ---- ops around the path: expert token counts, gating, routing with built-in quantisation, finalize ------------
namespace tab {

// out[e] = number of entries of the ascending int32 array `sorted` that are <= e (cumulative tokens per expert).
__global__ void __launch_bounds__(256) compute_expert_tokens_kernel(const int32_t* __restrict__ sorted, int n, int num_experts,
                                                                    int32_t* __restrict__ out) {
  for (int e = blockIdx.x * 256 + threadIdx.x; e < num_experts; e += gridDim.x * 256) {
    int lo = 0, hi = n;   // first index with sorted[idx] > e
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (sorted[mid] <= e) lo = mid + 1; else hi = mid;
    }
    out[e] = lo;
  }
}

// One warp per token: softmax over E <= 1024 logits held 32 per lane, then k rounds of a warp-shuffle arg-max
// (larger probability first, lower expert id on ties).  y [T, k] probabilities in the input dtype, expert_idx and
// row_idx int32 [T, k] with row_idx[t, j] = j*T + t.
constexpr int kGateMaxPerLane = 32;
template <typename T>
__global__ void __launch_bounds__(128) gating_topk_softmax_kernel(const T* __restrict__ x, const uint8_t* __restrict__ finished,
                                                                  int64_t tokens, int E, int k,
                                                                  T* __restrict__ y, int32_t* __restrict__ expert_idx,
                                                                  int32_t* __restrict__ row_idx) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (blockIdx.x * 128 + threadIdx.x) >> 5;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 4;
  for (int64_t t = warp_global; t < tokens; t += warps_total) {
    float v[kGateMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < E ? Elem<T>::to_f32(x[t * E + e]) : -INFINITY;
      m = fmaxf(m, v[i]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      v[i] = i * 32 + lane < E ? expf(v[i] - m) : 0.f;
      sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) v[i] = i * 32 + lane < E ? __fdiv_rn(v[i], sum) : -1.f;
    for (int j = 0; j < k; ++j) {
      float best = -2.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        if (v[i] > best) {   // ascending i keeps the lowest expert id among equal values of this lane
          best = v[i];
          best_e = i * 32 + lane;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < kGateMaxPerLane; ++i)
          if (i == (best_e >> 5)) v[i] = -1.f;   // taken
      }
      if (lane == 0) {
        y[t * k + j] = Elem<T>::from_f32(best);
        expert_idx[t * k + j] = (finished != nullptr && finished[t] != 0) ? E : best_e;   // a finished row points past the experts
        row_idx[t * k + j] = static_cast<int32_t>(j * tokens + t);
      }
    }
  }
}

// out[t] = sum_k scales[t,k] * (rows[src_to_dst[k*T + t]] + bias[expert[t,k]]) + skip1[t] + skip2[t]; fp32, ascending k.
template <typename T>
__global__ void __launch_bounds__(256) finalize_routing_kernel(const T* __restrict__ rows, const T* __restrict__ skip1,
                                                               const T* __restrict__ skip2, const T* __restrict__ bias,
                                                               const float* __restrict__ scales, const int32_t* __restrict__ src_to_dst,
                                                               const int32_t* __restrict__ expert, int64_t tokens, int K, int cols,
                                                               T* __restrict__ out) {
  extern __shared__ int s_meta[];  // [K] positions, [K] experts, [K] weights
  int* s_pos = s_meta;
  int* s_exp = s_meta + K;
  float* s_w = reinterpret_cast<float*>(s_meta + 2 * K);
  const int nchunk = cols >> 3;
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += 256) {
      s_pos[k] = src_to_dst[static_cast<int64_t>(k) * tokens + t];
      s_exp[k] = expert ? expert[t * K + k] : 0;
      s_w[k] = scales ? scales[t * K + k] : 1.f;
    }
    __syncthreads();
    for (int ch = threadIdx.x; ch < nchunk; ch += 256) {
      float acc[8];
      for (int k = 0; k < K; ++k) {
        float v[8];
        Elem<T>::load8(rows + static_cast<int64_t>(s_pos[k]) * cols + ch * 8, v);
        if (bias) {
          float b[8];
          Elem<T>::load8(bias + static_cast<int64_t>(s_exp[k]) * cols + ch * 8, b);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __fadd_rn(v[i], b[i]);
        }
        const float w = s_w[k];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float term = __fmul_rn(w, v[i]);
          acc[i] = k == 0 ? term : __fadd_rn(acc[i], term);
        }
      }
      if (skip1) {
        float v[8];
        Elem<T>::load8(skip1 + t * cols + ch * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
      }
      if (skip2) {
        float v[8];
        Elem<T>::load8(skip2 + t * cols + ch * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
      }
      Elem<T>::store8(out + t * cols + ch * 8, acc);
    }
  }
}

}  // namespace tab

extern "C" int tab_moe_compute_expert_tokens(const int32_t* sorted_experts, int64_t n, int64_t num_experts, int32_t* out,
                                             tab_stream_t stream) {
  if (n < 0 || num_experts <= 0 || n > (1LL << 30) || num_experts > (1LL << 24)) return fail(TAB_ERR_BAD_ARG, "compute_expert_tokens: n=%lld experts=%lld", (long long)n, (long long)num_experts);
  if (!out || (n > 0 && !sorted_experts)) return fail(TAB_ERR_BAD_ARG, "compute_expert_tokens: null pointer");
  compute_expert_tokens_kernel<<<grid_for((num_experts + 255) / 256, 4), 256, 0, as_stream(stream)>>>(sorted_experts, (int)n, (int)num_experts, out);
  return check_launch("compute_expert_tokens");
}

extern "C" int tab_moe_gating_top_k_softmax(const void* x, int dtype, const uint8_t* finished, int64_t tokens, int64_t num_experts,
                                            int64_t k, void* y, int32_t* expert_idx, int32_t* row_idx, tab_stream_t stream) {
  if (tokens < 0 || num_experts <= 0 || k <= 0 || k > num_experts) return fail(TAB_ERR_BAD_ARG, "gating_top_k_softmax: tokens=%lld experts=%lld k=%lld", (long long)tokens, (long long)num_experts, (long long)k);
  if (num_experts > 32 * kGateMaxPerLane) return fail(TAB_ERR_UNSUPPORTED, "gating_top_k_softmax: more than %d experts", 32 * kGateMaxPerLane);
  if (tokens == 0) return TAB_OK;
  if (!x || !y || !expert_idx || !row_idx) return fail(TAB_ERR_BAD_ARG, "gating_top_k_softmax: null pointer");
  const int grid = grid_for((tokens + 3) / 4, 8);
  cudaStream_t st = as_stream(stream);
  if (dtype == TAB_F32) gating_topk_softmax_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(x), finished, tokens, (int)num_experts, (int)k, static_cast<float*>(y), expert_idx, row_idx);
  else if (dtype == TAB_BF16) gating_topk_softmax_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), finished, tokens, (int)num_experts, (int)k, static_cast<__nv_bfloat16*>(y), expert_idx, row_idx);
  else if (dtype == TAB_F16) gating_topk_softmax_kernel<__half><<<grid, 128, 0, st>>>(static_cast<const __half*>(x), finished, tokens, (int)num_experts, (int)k, static_cast<__half*>(y), expert_idx, row_idx);
  else return fail(TAB_ERR_UNSUPPORTED, "gating_top_k_softmax: dtype %d (want 5, 6 or 15)", dtype);
  return check_launch("gating_top_k_softmax");
}

extern "C" int tab_moe_finalize_routing(const void* rows, int dtype, const void* skip1, const void* skip2, const void* bias,
                                        const float* scales, const int32_t* src_to_dst, const int32_t* expert_for_row, int64_t T,
                                        int64_t K, int64_t H, void* out, tab_stream_t stream) {
  if (T < 0 || K <= 0 || K > 1024 || H <= 0) return fail(TAB_ERR_BAD_ARG, "finalize_routing: T=%lld K=%lld H=%lld", (long long)T, (long long)K, (long long)H);
  if (T == 0) return TAB_OK;
  if (!rows || !src_to_dst || !out || (bias && !expert_for_row)) return fail(TAB_ERR_BAD_ARG, "finalize_routing: null pointer (bias needs expert_for_source_row)");
  if (H % 8 != 0 || !aligned16(rows) || !aligned16(out) || (skip1 && !aligned16(skip1)) || (skip2 && !aligned16(skip2)) || (bias && !aligned16(bias)))
    return fail(TAB_ERR_ALIGNMENT, "finalize_routing: H=%lld must be a multiple of 8 and pointers 16-byte aligned", (long long)H);
  cudaStream_t st = as_stream(stream);
  const int grid = grid_for(T, 8);
  const size_t smem = static_cast<size_t>(K) * 12;
  if (dtype == TAB_BF16)
    finalize_routing_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(rows), static_cast<const __nv_bfloat16*>(skip1), static_cast<const __nv_bfloat16*>(skip2), static_cast<const __nv_bfloat16*>(bias), scales, src_to_dst, expert_for_row, T, (int)K, (int)H, static_cast<__nv_bfloat16*>(out));
  else if (dtype == TAB_F16)
    finalize_routing_kernel<__half><<<grid, 256, smem, st>>>(static_cast<const __half*>(rows), static_cast<const __half*>(skip1), static_cast<const __half*>(skip2), static_cast<const __half*>(bias), scales, src_to_dst, expert_for_row, T, (int)K, (int)H, static_cast<__half*>(out));
  else if (dtype == TAB_F32)
    finalize_routing_kernel<float><<<grid, 256, smem, st>>>(static_cast<const float*>(rows), static_cast<const float*>(skip1), static_cast<const float*>(skip2), static_cast<const float*>(bias), scales, src_to_dst, expert_for_row, T, (int)K, (int)H, static_cast<float*>(out));
  else
    return fail(TAB_ERR_UNSUPPORTED, "finalize_routing: dtype %d (want 5, 6 or 15)", dtype);
  return check_launch("finalize_routing");
}

extern "C" int tab_moe_init_routing_v2(const void* x, int x_dtype, const int32_t* expert_idx, int64_t T, int64_t K, int64_t H,
                                       int64_t expert_lo, int64_t expert_hi, int quant_mode, int tokens_num_type, int row_idx_type,
                                       int64_t active_rows, const float* scale, int64_t scale_rows, void* expanded_x,
                                       int32_t* expanded_row_idx, int64_t* expert_tokens, float* expanded_scale, void* workspace,
                                       size_t workspace_bytes, tab_stream_t stream) {
  // Sort + (quantise or copy) + scatter are the dispatch sender's steps; this entry point adds the v2 outputs.
  if (quant_mode != -1 && quant_mode != 1) return fail(TAB_ERR_UNSUPPORTED, "init_routing_v2: quant_mode %d (want -1 or 1)", quant_mode);
  if ((tokens_num_type != 0 && tokens_num_type != 1) || (row_idx_type != 0 && row_idx_type != 1)) return fail(TAB_ERR_BAD_ARG, "init_routing_v2: bad type flag");
  const int64_t expert_num = expert_hi - expert_lo;
  size_t need = 0;
  int rc = tab_moe_dispatch_pack_workspace_bytes(T, K, expert_num, &need);
  if (rc != TAB_OK) return rc;
  const int64_t n = T * K;
  const size_t extra = static_cast<size_t>((n + expert_num) * 4 + 512);
  if (!workspace || workspace_bytes < need + extra) return fail(TAB_ERR_WORKSPACE, "init_routing_v2: workspace %zu < %zu bytes", workspace_bytes, need + extra);
  if (!expanded_row_idx || !expert_tokens || !expanded_scale) return fail(TAB_ERR_BAD_ARG, "init_routing_v2: null pointer");
  if (scale && quant_mode == -1 && scale_rows != T) return fail(TAB_ERR_BAD_ARG, "init_routing_v2: without quantisation `scale` holds one value per token");
  uint8_t* wsb = static_cast<uint8_t*>(workspace);
  int32_t* scatter_idx = reinterpret_cast<int32_t*>(wsb + need);               // f -> position
  int32_t* counts = scatter_idx + ((n + 63) / 64) * 64;
  int32_t* idx_out = row_idx_type == 1 ? expanded_row_idx : scatter_idx;
  // the pack kernel also writes the rows per expert as int64 counts or their running total
  rc = tab_moe_dispatch_pack_ex(x, x_dtype, expert_idx, T, K, H, expert_lo, expert_hi, /*drop_outside=*/1, nullptr,
                                quant_mode == 1 ? scale : nullptr, quant_mode == 1 ? scale_rows : 0,
                                quant_mode == -1 ? scale : nullptr, active_rows, quant_mode == 1 ? 2 : 0, expanded_x, expanded_scale,
                                idx_out, counts, expert_tokens, tokens_num_type, workspace, need, stream);
  if (rc != TAB_OK) return rc;
  cudaStream_t st = as_stream(stream);
  if (row_idx_type == 0 && n > 0) {
    // gather form: position -> source pair index, kept by the sort in its scratch (SortScratch::sorted_src); the pairs
    // of experts outside the range come after the kept ones
    SortScratch s = carve(workspace, n, expert_num + 1, true);
    cudaError_t e = cudaMemcpyAsync(expanded_row_idx, s.sorted_src, n * sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "init_routing_v2: copy: %s", cudaGetErrorString(e));
  }
  return check_launch("init_routing_v2", 0);   // the kernels were counted by the calls above
}

// ---- npu_moe_gating_top_k: softmax or sigmoid scores, optional selection bias, group-limited top-k ----------------
namespace tab {

__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

// One warp per token; E <= 1024 scores, 32 per lane (element e = i*32 + lane); group_count <= 32 contiguous groups.
template <typename T>
__global__ void __launch_bounds__(128) gating_topk_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                                          const uint8_t* __restrict__ finished, int64_t tokens, int E,
                                                          int k, int k_group, int group_count, int group_select_mode, int norm_type,
                                                          float scaling, float eps, T* __restrict__ y, int32_t* __restrict__ expert_idx,
                                                          float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (blockIdx.x * 128 + threadIdx.x) >> 5;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * 4;
  const int G = E / group_count;
  const float kGone = -INFINITY;
  for (int64_t t = warp_global; t < tokens; t += warps_total) {
    float sc[kGateMaxPerLane], sel[kGateMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      sc[i] = e < E ? Elem<T>::to_f32(x[t * E + e]) : -INFINITY;
      m = fmaxf(m, sc[i]);
    }
    if (norm_type != 1) {
      m = warp_max(m);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        sc[i] = i * 32 + lane < E ? expf(sc[i] - m) : 0.f;
        sum += sc[i];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) sc[i] = __fdiv_rn(sc[i], sum);
    } else {
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) sc[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-sc[i])));
    }
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < E) {
        if (out) out[t * E + e] = sc[i];
        sel[i] = bias ? __fadd_rn(sc[i], Elem<T>::to_f32(bias[e])) : sc[i];
      } else {
        sel[i] = kGone;
      }
    }
    if (group_count > 1) {
      // score of group g lands in lane g: its maximum, or the sum of its two largest selection scores
      float gscore = kGone;
      for (int g = 0; g < group_count; ++g) {
        float b1 = kGone;
        int i1 = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kGateMaxPerLane; ++i) {
          const int e = i * 32 + lane;
          if (e < E && e / G == g && sel[i] > b1) {
            b1 = sel[i];
            i1 = e;
          }
        }
        warp_argmax(b1, i1);
        float s = b1;
        if (group_select_mode == 1) {
          float b2 = kGone;
          int i2 = 0x7fffffff;
#pragma unroll
          for (int i = 0; i < kGateMaxPerLane; ++i) {
            const int e = i * 32 + lane;
            if (e < E && e / G == g && e != i1 && sel[i] > b2) {
              b2 = sel[i];
              i2 = e;
            }
          }
          warp_argmax(b2, i2);
          s = __fadd_rn(b1, b2);
        }
        if (lane == g) gscore = s;
      }
      unsigned keep = 0u;
      for (int j = 0; j < k_group; ++j) {
        float v = gscore;
        int gi = lane < group_count ? lane : 0x7fffffff;
        if (lane >= group_count) v = kGone;
        warp_argmax(v, gi);
        keep |= 1u << gi;
        if (lane == gi) gscore = kGone;
      }
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        const int e = i * 32 + lane;
        if (e < E && !((keep >> (e / G)) & 1u)) sel[i] = kGone;
      }
    }
    float ysum = 0.f;
    float mine = 0.f;       // lane j keeps the j-th selected score (k <= 32) for the normalisation pass
    int mine_e = 0;
    for (int j = 0; j < k; ++j) {
      float best = kGone;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        if (sel[i] > best) {
          best = sel[i];
          best_e = i * 32 + lane;
        }
      }
      warp_argmax(best, best_e);
      float score = 0.f;
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        if ((best_e & 31) == lane && i == (best_e >> 5)) {
          score = sc[i];
          sel[i] = kGone;
        }
      }
      score = __shfl_sync(0xffffffffu, score, best_e & 31);
      ysum = __fadd_rn(ysum, score);
      if (lane == j) {
        mine = score;
        mine_e = best_e;
      }
    }
    if (lane < k) {
      float v = mine;
      if (norm_type != 0) v = __fdiv_rn(v, __fadd_rn(ysum, eps));   // sigmoid scores, or softmax renormalised over the k
      v = __fmul_rn(v, scaling);
      y[t * k + lane] = Elem<T>::from_f32(v);
      expert_idx[t * k + lane] = (finished != nullptr && finished[t] != 0) ? E : mine_e;
    }
  }
}

}  // namespace tab

extern "C" int tab_moe_gating_top_k(const void* x, const void* bias, const uint8_t* finished, int dtype, int64_t tokens,
                                    int64_t num_experts, int64_t k,
                                    int64_t k_group, int64_t group_count, int group_select_mode, int norm_type,
                                    float routed_scaling_factor, float eps, void* y, int32_t* expert_idx, float* out,
                                    tab_stream_t stream) {
  if (tokens < 0 || num_experts <= 0 || k <= 0 || k > num_experts || k > 32)
    return fail(TAB_ERR_BAD_ARG, "gating_top_k: tokens=%lld experts=%lld k=%lld (k must be in [1, 32])", (long long)tokens, (long long)num_experts, (long long)k);
  if (num_experts > 32 * kGateMaxPerLane) return fail(TAB_ERR_UNSUPPORTED, "gating_top_k: more than %d experts", 32 * kGateMaxPerLane);
  if (group_count < 1 || group_count > 32 || num_experts % group_count != 0 || k_group < 1 || k_group > group_count ||
      k > k_group * (num_experts / group_count))
    return fail(TAB_ERR_BAD_ARG, "gating_top_k: group_count=%lld k_group=%lld do not fit %lld experts and k=%lld", (long long)group_count, (long long)k_group, (long long)num_experts, (long long)k);
  if ((group_select_mode != 0 && group_select_mode != 1) || norm_type < 0 || norm_type > 2)
    return fail(TAB_ERR_UNSUPPORTED, "gating_top_k: group_select_mode must be 0 or 1 and norm_type 0, 1 or 2");
  if (group_select_mode == 1 && num_experts / group_count < 2) return fail(TAB_ERR_BAD_ARG, "gating_top_k: top-2 group score needs groups of at least two experts");
  if (tokens == 0) return TAB_OK;
  if (!x || !y || !expert_idx) return fail(TAB_ERR_BAD_ARG, "gating_top_k: null pointer");
  const int grid = grid_for((tokens + 3) / 4, 8);
  cudaStream_t st = as_stream(stream);
#define TAB_GATE_LAUNCH(TYPE)                                                                                                     \
  gating_topk_kernel<TYPE><<<grid, 128, 0, st>>>(static_cast<const TYPE*>(x), static_cast<const TYPE*>(bias), finished, tokens, (int)num_experts, \
                                                 (int)k, (int)k_group, (int)group_count, group_select_mode, norm_type,           \
                                                 routed_scaling_factor, eps, static_cast<TYPE*>(y), expert_idx, out)
  if (dtype == TAB_F32) TAB_GATE_LAUNCH(float);
  else if (dtype == TAB_BF16) TAB_GATE_LAUNCH(__nv_bfloat16);
  else if (dtype == TAB_F16) TAB_GATE_LAUNCH(__half);
  else return fail(TAB_ERR_UNSUPPORTED, "gating_top_k: dtype %d (want 5, 6 or 15)", dtype);
#undef TAB_GATE_LAUNCH
  return check_launch("gating_top_k");
}
