/*
 * torchair-b200 C ABI: the device side of the W8A8 expert-parallel MoE path on NVIDIA B200 (sm_100a).
 *
 * The shared library libtorchair_b200.so exports exactly the functions declared here.  They are what a
 * foreign-function binding of the reference's operators for this path would call in place of the closed
 * vendor kernels.  Each declaration cites the reference interface it stands in for (paths are inside the
 * Ascend/torchair project; "converter" = python/torchair/_ge_concrete_graph/ge_converter/custom).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless the comment says "host".
 *   - Nothing is allocated, freed or synchronised inside a call; all work is enqueued on `stream`
 *     (a cudaStream_t), so calls are legal during CUDA-graph capture.  Scratch memory is passed in as
 *     `workspace`; the matching *_workspace_bytes function says how much is needed.
 *   - Return value: 0 on success, a negative tab_status otherwise.  tab_last_error() returns a message for
 *     the calling thread's most recent failure.  No call aborts or throws.
 *   - dtype arguments use the c10::ScalarType integers the reference's converters use
 *     (python/torchair/ge/_ge_graph.py:215-270): 1 int8, 3 int32, 4 int64, 5 float16, 6 float32, 15 bfloat16.
 *   - Row-major, contiguous tensors; rows of 8-bit data must be 16-byte multiples.
 */
#ifndef TAB_API_H_
#define TAB_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tab_stream_t; /* cudaStream_t */

#if defined(__GNUC__)
#define TAB_API __attribute__((visibility("default")))
#else
#define TAB_API
#endif

enum tab_status {
  TAB_OK = 0,
  TAB_ERR_BAD_ARG = -1,     /* null pointer, negative size, inconsistent shapes */
  TAB_ERR_UNSUPPORTED = -2, /* dtype / mode outside the path */
  TAB_ERR_ALIGNMENT = -3,   /* pointer or row pitch not 16-byte aligned */
  TAB_ERR_WORKSPACE = -4,   /* workspace too small */
  TAB_ERR_CUDA = -5,        /* a CUDA runtime/driver call failed; message holds its text */
  TAB_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up (read back via tab_gmm_status) */
};

enum tab_dtype { TAB_I8 = 1, TAB_I32 = 3, TAB_I64 = 4, TAB_F16 = 5, TAB_F32 = 6, TAB_BF16 = 15 };

/* Library version (major*10000 + minor*100 + patch).  Nearest reference analogue: the pybind module
 * `_torchair` (torchair/core/npu_wrapper.cpp:28-84). */
TAB_API int tab_version(void);

/* Number of kernels this library has enqueued so far in this process, over all devices and streams (a launch
 * recorded into a CUDA graph during capture counts once, its replays do not pass through the library).  For
 * accounting in benchmarks; no counterpart in the reference. */
TAB_API long long tab_launch_count(void);

/* Message of the calling thread's last failing call.  Stands in for tng::Status -> RuntimeError
 * (torchair/core/torchair.cpp:98-120). */
TAB_API const char* tab_last_error(void);

/* ---------------------------------------------------------------------------------------------------
 * npu_dynamic_quant  (converter npu_dynamic_quant.py:8-40 -> DynamicQuant, nn_quantize.h:28-54)
 * x [rows, cols] of x_dtype (5, 6 or 15); smooth [cols] of x_dtype or NULL.
 * y int8 [rows, cols]; scale fp32 [rows] = amax(|x*smooth|)/127; y = clamp(rint(v/scale), +-127).
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_dynamic_quant(const void* x, int x_dtype, const void* smooth, int64_t rows, int64_t cols,
                      int8_t* y, float* scale, tab_stream_t stream);

/* tab_quant_status: host-side; synchronises `stream` and copies the status word of the row kernels that stream rows
 * through shared memory (tab_dynamic_quant, tab_dequant_swiglu_quant): 0, or 1 after a bounded wait for a bulk copy gave
 * up (TAB_ERR_TIMEOUT); the CTA then stops and leaves its remaining rows unwritten.  No counterpart in the reference. */
TAB_API int tab_quant_status(int* status_host, tab_stream_t stream);

/* tab_selftest_reciprocal: adds to *mismatches (device uint64, zeroed by the caller) the number of significands, out
 * of all 2^23 at the binary exponent `exponent`, for which the reciprocal used inside SwiGLU (hardware seed + one
 * Newton step) differs from the IEEE reciprocal, plus those for which the row quantiser's short forms of amax / 127
 * and of its reciprocal differ from IEEE division.  Results are reproducible on a CPU exactly when this is 0; the GPU
 * tests check it.  No counterpart in the reference. */
TAB_API int tab_selftest_reciprocal(int exponent, unsigned long long* mismatches, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_swiglu  (converter npu_swiglu.py:8-14 -> SwiGlu), last-dimension split only.
 * x [rows, cols] (cols even) of dtype 5, 6 or 15; y [rows, cols/2] = silu(x[:, :cols/2]) * x[:, cols/2:].
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_swiglu(const void* x, int dtype, int64_t rows, int64_t cols, void* y, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_dequant_swiglu_quant, dynamic mode (converter npu_dequant_swiglu_quant.py:5-64 ->
 * DequantSwigluQuant, experiment_ops.h:3764-3811).
 * x int32 [rows, cols]; weight_scale fp32 [ws_groups, cols] (ws_groups == 1: one row for all) or NULL;
 * activation_scale fp32 [rows] or NULL; group_index int64 [num_groups] per-group row COUNTS or NULL
 * (required when ws_groups > 1; rows past their sum give y = 0, scale = 0).
 * y int8 [rows, cols/2]; scale fp32 [rows].
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_dequant_swiglu_quant(const int32_t* x, const float* weight_scale, int64_t ws_groups,
                             const float* activation_scale, const int64_t* group_index, int64_t num_groups,
                             int activate_left, int64_t rows, int64_t cols, int8_t* y, float* scale,
                             tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_moe_init_routing  (converter moe_init_routing.py:10-21 -> MoeInitRouting, experiment_ops.h:2111-2134)
 * x [T, H] of x_dtype; row_idx, expert_idx int32 [T, K]; expert ids must lie in [0, expert_bound).
 * expanded_x [min(T, active_num)*K, H]; expanded_row_idx, expanded_expert_idx int32 [T*K].
 * Stable counting sort of the T*K pairs by expert id (ties by flattened index), row gather.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_init_routing_workspace_bytes(int64_t T, int64_t K, int64_t expert_bound, size_t* bytes);
TAB_API int tab_moe_init_routing(const void* x, int x_dtype, const int32_t* row_idx, const int32_t* expert_idx,
                         int64_t T, int64_t K, int64_t H, int64_t active_num, int64_t expert_bound,
                         void* expanded_x, int32_t* expanded_row_idx, int32_t* expanded_expert_idx,
                         void* workspace, size_t workspace_bytes, tab_stream_t stream);

/* tab_routing_status: host-side; synchronises `stream`, copies the routing kernels' device status word to
 * *status_host and clears it.  Bit 0: an expert id outside [0, bound) reached a sort (tab_moe_init_routing,
 * tab_moe_init_routing_static, tab_moe_dispatch_pack, tab_moe_init_routing_v2) and was clamped to the nearest valid
 * id; bit 1: a row_idx value outside [0, T*K) was skipped.  Neither accesses memory out of range; a non-zero word
 * returns TAB_ERR_BAD_ARG with a message.  The reference's IR prototype (MoeInitRouting,
 * experiment_ops.h:2111-2134) states no behaviour for ids out of range; this library clamps and reports. */
TAB_API int tab_routing_status(int* status_host, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * tab_moe_init_routing_static: npu_moe_init_routing for callers that cannot hand over scratch memory.
 * No counterpart in the reference: it exists for hosts that bind this library without a device allocator of
 * their own -- a plugin running inside another framework's memory pool, a real-time loop that fixed its
 * allocations at start-up -- and so can neither cudaMalloc a workspace nor ask torch for one.  Inputs and
 * outputs are still the caller's; the sort's scratch is a 256 KiB array inside the library's device image,
 * present once on every GPU that loads the library until the process exits.
 * Limits: T*K <= 32768 and expert_bound <= 512; larger problems are rejected with TAB_ERR_UNSUPPORTED (use
 * tab_moe_init_routing with a workspace).  The call itself allocates and frees nothing.
 * The first call on each device looks up the array's device address (with that device current); make that
 * first call before starting any stream capture.  All calls on a device share the one array: calls that may
 * overlap on the GPU (different streams, no ordering between them) race on it and must be serialised by the
 * caller.  Same arguments and results as tab_moe_init_routing otherwise.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_init_routing_static(const void* x, int x_dtype, const int32_t* row_idx, const int32_t* expert_idx,
                                int64_t T, int64_t K, int64_t H, int64_t active_num, int64_t expert_bound,
                                void* expanded_x, int32_t* expanded_row_idx, int32_t* expanded_expert_idx,
                                tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_moe_distribute_dispatch, sender side (converter moe_distribute_dispatch.py:4-45 ->
 * MoeDistributeDispatch).  Sorts this rank's T*K copies by global expert id (stable), quantises every
 * token once (quant_mode 2: int8 rows + fp32 scales; quant_mode 0: rows keep x_dtype, scales = 0) and
 * writes the copies in sorted order:
 *   send_rows [T*K, H], send_scales fp32 [T*K], expand_idx int32 [T*K] (position of pair t*K+k),
 *   expert_counts int32 [num_experts] (copies per global expert); expert_token_nums int64 [num_experts] (NULL to
 *   skip) = the same counts (nums_type 1) or their running total (0), the form the grouped GEMM's group_list takes.
 * With one rank this is the whole dispatch: send_rows is expand_x and expert_token_nums the operator's output.
 *
 * tab_moe_dispatch_pack_ex adds the optional arguments of the operators built on this step (decisions where the
 * reference gives a name only):
 *   expert_lo, expert_hi  experts [lo, hi) are kept and numbered from 0 (num_experts = hi - lo in every output).  An id
 *                         outside the range is dropped when drop_outside != 0 (active_expert_range of
 *                         npu_moe_init_routing_v2, npu_moe_init_routing_v2.py:55,81; ids >= moe_expert_num of the
 *                         second-generation dispatch name special experts that are not sent,
 *                         moe_distribute_dispatch_v2.py:15-18), else clamped into the range and reported.
 *   x_active_mask         bytes [T] or NULL (moe_distribute_dispatch.py:14,31): tokens whose byte is 0 send nothing.
 *   smooth                fp32 [smooth_rows, H] or NULL (`scales` of dispatch, `scale` of init_routing_v2 with dynamic
 *                         quantisation): copy (t, k) is quantised after the fp32 product x[t] * smooth[expert - lo]
 *                         (smooth_rows == num_experts) or x[t] * smooth[0] (smooth_rows == 1), each copy with its own
 *                         scale.  quant_mode 2 only.
 *   passthrough_scale     fp32 [T] or NULL, quant_mode 0 only: send_scales of a copy = the value of its token.
 *   pos_limit             > 0: copies at sorted positions >= pos_limit get no row (active_num); 0 = no limit.
 * Dropped pairs get expand_idx = -1 and no row; they are not counted.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_dispatch_pack_workspace_bytes(int64_t T, int64_t K, int64_t num_experts, size_t* bytes);
TAB_API int tab_moe_dispatch_pack_ex(const void* x, int x_dtype, const int32_t* expert_ids, int64_t T, int64_t K, int64_t H,
                             int64_t expert_lo, int64_t expert_hi, int drop_outside, const uint8_t* x_active_mask,
                             const float* smooth, int64_t smooth_rows, const float* passthrough_scale,
                             int64_t pos_limit, int quant_mode, void* send_rows, float* send_scales,
                             int32_t* expand_idx, int32_t* expert_counts, int64_t* expert_token_nums, int nums_type,
                             void* workspace, size_t workspace_bytes, tab_stream_t stream);
TAB_API int tab_moe_dispatch_pack(const void* x, int x_dtype, const int32_t* expert_ids, int64_t T, int64_t K,
                          int64_t H, int64_t num_experts, int quant_mode, void* send_rows,
                          float* send_scales, int32_t* expand_idx, int32_t* expert_counts,
                          int64_t* expert_token_nums, int nums_type,
                          void* workspace, size_t workspace_bytes, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_moe_distribute_dispatch, receiver side, and npu_moe_distribute_combine, expert side
 * (converters moe_distribute_dispatch.py:4-45, moe_distribute_combine.py:4-60).
 * recv_counts int32 [R, E_l]: rows this rank received from source rank s for its local expert e.  The
 * wire buffer holds them source-major: rank s's block starts at row s*slot_rows (slot_rows > 0: fixed
 * slots) or at the running total (slot_rows == 0: packed).  The expert-side buffer orders rows by
 * (local expert, source rank).
 *   tab_moe_exchange_plan   writes  plan int32 [2*R*E_l + 1] (row offsets on both sides),
 *                           expert_token_nums int64 [E_l] (counts if nums_type == 1 else cumsum),
 *                           ep_recv_count int32 [E_l*R] (count of expert e from rank s at e*R+s).
 *   tab_moe_exchange_rows   direction 0: wire -> expert order (rows + optional fp32 scales);
 *                           direction 1: expert order -> wire.  dst has dst_rows rows; rows of dst not
 *                           covered by the plan are zero-filled when zero_fill != 0.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_exchange_plan(const int32_t* recv_counts, int64_t R, int64_t E_l, int64_t slot_rows,
                          int nums_type, int32_t* plan, int64_t* expert_token_nums,
                          int32_t* ep_recv_count, tab_stream_t stream);
TAB_API int tab_moe_exchange_rows(const void* src, const float* src_scales, const int32_t* plan, int64_t R,
                          int64_t E_l, int64_t slot_rows, int direction, int64_t row_bytes,
                          int64_t dst_rows, int zero_fill, void* dst, float* dst_scales,
                          tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_moe_distribute_dispatch / npu_moe_distribute_combine over peer memory, for the GPUs of one node
 * (converters moe_distribute_dispatch.py:4-45, moe_distribute_combine.py:4-60; the reference's kernels also
 * communicate from inside the operator).  Rows are stored straight into the destination GPU's receive
 * buffer; no library collective and no host read is involved, so the exchange can be captured in a CUDA
 * graph.  The caller provides peer-mapped (symmetric) memory: `peer_*` arguments are DEVICE arrays of R
 * device pointers, one per rank (entry r points into rank r's memory, this rank's own entry included).
 *   layout on every rank: recv [R][slot_rows][row_bytes + 16] (the 16-byte tail carries the fp32 scale),
 *   counts int32 [R][E_l], ret [R][slot_rows][row_bytes], flag arrays uint64 [R], counters uint64.
 *   tab_ep_signal      stores (counter + 1) into peer_flags[r] for every r, then counter += 1.
 *   tab_ep_wait        waits (bounded, ~2 s) until flags[s] >= counter + pre_increment for every s, then
 *                      counter += 1; on expiry writes `code` into *status (device int) and continues.
 *   tab_ep_send_rows   sender: row p of the expert-sorted rows goes to rank d = owner of its expert, slot
 *                      [my_rank][p - first row of d]; per-expert counts go to peer_counts; expand_idx_slot[f]
 *                      = d*slot_rows + offset is the position at which the combined row comes back.  A row whose
 *                      offset does not fit the slot (counts and slot_rows disagree) is not sent; `code` is then
 *                      written to the device word `status` (the word tab_ep_wait reports into).
 *   tab_ep_unpack_rows receiver: slot records -> rows in (local expert, source) order + scales; `plan` from
 *                      tab_moe_exchange_plan(counts, R, E_l, slot_rows, ...).
 *   tab_ep_return_rows expert side of combine: outputs go back to slot [my_rank][send offset] of the source
 *                      rank's `ret` buffer; the source then runs tab_moe_combine on its ret buffer with
 *                      expand_idx_slot.
 *   tab_ep_return_plan the addresses tab_ep_return_rows would copy to, one per expert-output row (0 past the
 *                      total and for a row whose offset does not fit its slot), as the row table of
 *                      tab_grouped_matmul_w8a8_scatter: the down GEMM then stores its rows into the source ranks'
 *                      `ret` buffers itself and no copy kernel runs.
 * Fused forms that save launches on the decode path (same data movement, same buffers):
 *   tab_ep_send_rows with ack_flags != NULL: every CTA first checks, bounded, that each source's acknowledgement
 *                      flag has reached *ack_counter (the peers have copied the previous rows out); the counter is
 *                      advanced by the tab_ep_signal_wait that follows (its bump_counter).  On expiry ack_code goes to
 *                      *status and the rows are sent all the same.
 *   tab_ep_signal_wait tab_ep_signal on (peer_flags, sig_counter) followed by tab_ep_wait with pre_increment = 1 on
 *                      (flags, wait_counter) in one launch; *bump_counter += 1 when given.
 *   tab_ep_unpack_rows_fused  tab_moe_exchange_plan + tab_ep_unpack_rows in one launch (every CTA derives the offsets
 *                      from recv_counts int32 [R, E_l]); rows past the received total are left untouched; when
 *                      ack_peer_flags != NULL the CTA that finishes last performs the tab_ep_signal on
 *                      (ack_peer_flags, ack_sig_counter); done_counter: a zero-initialised device uint32 of the caller.
 *   tab_ep_return_plan_fused  tab_moe_exchange_plan + tab_ep_return_plan in one launch from ep_send_counts int32
 *                      [E_l, R]; when ack_flags != NULL its first CTA also performs tab_ep_wait(pre_increment = 0) on
 *                      (ack_flags, ack_counter) with ack_code.
 * Every flag wait is bounded (TAB_EP_WAIT_MS in the environment, read once; default 2000 ms).
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_ep_signal(void* const* peer_flags, void* counter, int64_t R, tab_stream_t stream);
TAB_API int tab_ep_wait(const void* flags, void* counter, int64_t R, int pre_increment, int* status, int code,
                tab_stream_t stream);
TAB_API int tab_ep_send_rows(const void* rows, const float* scales, const int32_t* expert_counts,
                     const int32_t* expand_idx, int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes,
                     int64_t M, int64_t my_rank, void* const* peer_recv, void* const* peer_counts,
                     int32_t* expand_idx_slot, int* status, int code, const void* ack_flags,
                     const void* ack_counter, int ack_code, tab_stream_t stream);
TAB_API int tab_ep_unpack_rows(const void* recv, const int32_t* plan, int64_t R, int64_t E_l, int64_t row_bytes,
                       int64_t dst_rows, int zero_fill, void* dst, float* dst_scales, tab_stream_t stream);
TAB_API int tab_ep_return_rows(const void* y, const int32_t* plan, int64_t R, int64_t E_l, int64_t slot_rows,
                       int64_t row_bytes, int64_t max_rows, int64_t my_rank, void* const* peer_ret,
                       tab_stream_t stream);

TAB_API int tab_ep_return_plan(const int32_t* plan, int64_t R, int64_t E_l, int64_t slot_rows, int64_t row_bytes,
                       int64_t max_rows, int64_t my_rank, void* const* peer_ret, uint64_t* row_dst,
                       tab_stream_t stream);
TAB_API int tab_ep_signal_wait(void* const* peer_flags, void* sig_counter, const void* flags, void* wait_counter,
                       int64_t R, int* status, int code, void* bump_counter, tab_stream_t stream);
TAB_API int tab_ep_unpack_rows_fused(const void* recv, const int32_t* recv_counts, int64_t R, int64_t E_l,
                             int64_t slot_rows, int64_t row_bytes, int64_t dst_rows, int nums_type, void* dst,
                             float* dst_scales, int64_t* expert_token_nums, int32_t* ep_recv_count,
                             void* const* ack_peer_flags, void* ack_sig_counter, void* done_counter,
                             tab_stream_t stream);
TAB_API int tab_ep_return_plan_fused(const int32_t* ep_send_counts, int64_t R, int64_t E_l, int64_t slot_rows,
                             int64_t row_bytes, int64_t max_rows, int64_t my_rank, void* const* peer_ret,
                             uint64_t* row_dst, const void* ack_flags, void* ack_counter, int* status, int ack_code,
                             tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_moe_distribute_combine, receiving side (converter moe_distribute_combine.py:4-60 ->
 * MoeDistributeCombine): out[t] = sum_k expert_scales[t,k] * rows[expand_idx[t*K+k]] (+ shared[t]),
 * fp32 accumulation in ascending k, one rounding to dtype (5 or 15).
 * rows [*, H]; expand_idx int32 [T*K]; expert_scales fp32 [T, K]; shared [T, H] or NULL; out [T, H].
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_combine(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                    const void* shared, int64_t T, int64_t K, int64_t H, void* out, tab_stream_t stream);
/* tab_moe_combine_ex: the same with the optional inputs (decisions where the converters give names only):
 *   x_active_mask bytes [T] or NULL (moe_distribute_combine.py:17): a 0 byte gives an all-zero output row;
 *   a negative expand_idx entry (a pair that was not dispatched) contributes 0;
 *   special experts of the second-generation operator (moe_distribute_combine_v2.py:17-20,47-50): a pair whose
 *   expert_ids entry (int32 [T, K]) is num_experts + s stands for a row formed here -- s < zero_expert_num: 0; the next
 *   copy_expert_num: the token itself, ori_x [T, H]; the next const_expert_num (index c): const_expert_alpha_1[c] *
 *   ori_x[t] + const_expert_alpha_2[c] * const_expert_v[c] ([const_expert_num, H] each, of `dtype`), two fp32 products
 *   and one fp32 sum per element -- which then enters the weighted sum like a gathered row. */
TAB_API int tab_moe_combine_ex(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                       const void* shared, int64_t T, int64_t K, int64_t H, void* out, const uint8_t* x_active_mask,
                       const int32_t* expert_ids, int64_t num_experts, int64_t zero_expert_num, int64_t copy_expert_num,
                       int64_t const_expert_num, const void* ori_x, const void* const_expert_alpha_1,
                       const void* const_expert_alpha_2, const void* const_expert_v, tab_stream_t stream);
/* tab_moe_combine_ack: tab_moe_combine_ex as the last step of a combine over peer memory (tab_ep_* below): when every CTA has
 *   read its rows, the last one stores the next sequence number (ack_sig_counter + 1, device counter, updated) into the flag
 *   slots ack_peer_flags[0..ack_ranks) of the peers, telling them that their stores into this rank's return buffer may go
 *   on; done_counter is a zero-initialised device word the CTAs count in (it is zero again afterwards).  Saves the
 *   separate tab_ep_signal launch.  T must be positive. */
TAB_API int tab_moe_combine_ack(const void* rows, int dtype, const int32_t* expand_idx, const float* expert_scales,
                        const void* shared, int64_t T, int64_t K, int64_t H, void* out, const uint8_t* x_active_mask,
                        const int32_t* expert_ids, int64_t num_experts, int64_t zero_expert_num, int64_t copy_expert_num,
                        int64_t const_expert_num, const void* ori_x, const void* const_expert_alpha_1,
                        const void* const_expert_alpha_2, const void* const_expert_v, void* const* ack_peer_flags,
                        void* ack_sig_counter, void* done_counter, int64_t ack_ranks, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * Operators next to the path.
 *
 * npu_moe_compute_expert_tokens (converter npu_moe_compute_expert_tokens.py:4-11 -> MoeComputeExpertTokens):
 *   sorted_experts int32 [n] ascending; out int32 [num_experts], out[e] = number of entries <= e.
 *
 * npu_moe_gating_top_k_softmax (converter moe_gating_top_k_softmax.py:9-19 -> MoeGatingTopKSoftmax,
 *   experiment_ops.h:2222-2241): softmax over the experts in fp32, then the k largest
 *   (ties: lower expert id).  x [tokens, num_experts] of dtype 5, 6 or 15 (num_experts <= 1024);
 *   y [tokens, k] same dtype; expert_idx, row_idx int32 [tokens, k], row_idx[t, j] = j*tokens + t.
 *   finished: bytes [tokens] or NULL (moe_gating_top_k_softmax.py:10-19); decision: a row whose byte is non-zero
 *   reports expert_idx = num_experts in every slot (an id past the experts, which the routing ops drop or clamp),
 *   y and row_idx as for any other row.  The same argument of tab_moe_gating_top_k serves
 *   npu_moe_gating_top_k_softmax_v2.
 *
 * npu_moe_finalize_routing (converter npu_moe_finalize_routing.py:21-41 -> MoeFinalizeRouting(V2)), drop_pad_mode 0:
 *   out[t] = sum_k scales[t,k] * (rows[src_to_dst[k*T + t]] + bias[expert_for_row[t,k]]) + skip1[t] + skip2[t];
 *   fp32 accumulation in ascending k, one rounding.  rows [*, H], skip1/skip2 [T, H], bias [E, H] of `dtype`
 *   (5, 6 or 15) or NULL; scales fp32 [T, K] or NULL (= 1); src_to_dst int32 [K*T]; expert_for_row int32 [T, K].
 *
 * npu_moe_init_routing_v2 (converter npu_moe_init_routing_v2.py:41-95 -> MoeInitRoutingV3, experiment_ops.h:2137-2192),
 *   dropless: stable sort of the T*K pairs (flattened index f = t*K + k) by expert id, rows copied (quant_mode -1)
 *   or quantised to int8 (quant_mode 1).  Experts [expert_lo, expert_hi) are kept (active_expert_range; expert_num
 *   below = expert_hi - expert_lo); pairs of other experts get no row and sort behind the kept ones.
 *   expanded_x [T*K, H], of which only rows at positions < active_rows are written when active_rows > 0 (active_num);
 *   expanded_row_idx int32 [T*K] (row_idx_type 0: sorted position -> f; 1: f -> sorted position, -1 for a pair that
 *   was not kept); expert_tokens int64 [expert_num] counts (tokens_num_type 1) or cumulative sums (0);
 *   expanded_scale fp32 [T*K].  scale: quant_mode -1: fp32 [T] (scale_rows == T), copied to expanded_scale of the
 *   token's copies (zero when NULL); quant_mode 1: fp32 smooth scales [expert_num, H] or [1, H] (scale_rows) applied
 *   before the per-copy quantisation, or NULL (one quantisation per token).
 *   Workspace: tab_moe_dispatch_pack_workspace_bytes(T, K, expert_num) + 4*(T*K + expert_num) + 1024 bytes.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_moe_compute_expert_tokens(const int32_t* sorted_experts, int64_t n, int64_t num_experts, int32_t* out,
                                  tab_stream_t stream);
TAB_API int tab_moe_gating_top_k_softmax(const void* x, int dtype, const uint8_t* finished, int64_t tokens,
                                 int64_t num_experts, int64_t k, void* y, int32_t* expert_idx, int32_t* row_idx,
                                 tab_stream_t stream);
 /* npu_moe_gating_top_k (converter npu_moe_gating_top_k.py:4-22 -> MoeGatingTopK, experiment_ops.h:3722-3761):
  * scores = softmax(x) (norm_type 0 and 2) or sigmoid(x) (1) in fp32; selection score = scores + bias; with group_count > 1 the
  * experts form contiguous groups, each scored by its maximum (group_select_mode 0) or by the sum of its two largest
  * selection scores (1), and only the k_group best groups stay eligible; the k best eligible experts are taken (ties:
  * lower id).  y [tokens, k] = the selected scores without bias, for norm_type 1 and 2 divided by (their sum + eps), times
  * routed_scaling_factor; expert_idx int32 [tokens, k]; out fp32 [tokens, experts] = all scores (NULL to skip).
  * num_experts <= 1024, k <= 32, group_count <= 32.  norm_type 2 with no bias and one group is
 * npu_moe_gating_top_k_softmax_v2 with renorm = 1 (converter npu_moe_gating_top_k_softmax_v2.py:9-23 ->
 * MoeGatingTopKSoftmaxV2, experiment_ops.h:2243-2265); norm_type 0 is its renorm = 0, `out` its softmax_result. */
TAB_API int tab_moe_gating_top_k(const void* x, const void* bias, const uint8_t* finished, int dtype, int64_t tokens,
                         int64_t num_experts, int64_t k,
                         int64_t k_group, int64_t group_count, int group_select_mode, int norm_type,
                         float routed_scaling_factor, float eps, void* y, int32_t* expert_idx, float* out,
                         tab_stream_t stream);
TAB_API int tab_moe_finalize_routing(const void* rows, int dtype, const void* skip1, const void* skip2, const void* bias,
                             const float* scales, const int32_t* src_to_dst, const int32_t* expert_for_row, int64_t T,
                             int64_t K, int64_t H, void* out, tab_stream_t stream);
TAB_API int tab_moe_init_routing_v2(const void* x, int x_dtype, const int32_t* expert_idx, int64_t T, int64_t K, int64_t H,
                            int64_t expert_lo, int64_t expert_hi, int quant_mode, int tokens_num_type, int row_idx_type,
                            int64_t active_rows, const float* scale, int64_t scale_rows, void* expanded_x,
                            int32_t* expanded_row_idx, int64_t* expert_tokens, float* expanded_scale, void* workspace,
                            size_t workspace_bytes, tab_stream_t stream);

/* ---------------------------------------------------------------------------------------------------
 * npu_grouped_matmul, W8A8 (converter grouped_matmul.py:210-365 -> GroupedMatmul,
 * experiment_ops.h:3616-3652).
 *
 * tab_prepack_weight_i8: one-off relayout of weight int8 [E, Kd, N] (the operator's layout, N contiguous)
 *   into packed int8 [E, N, Kd] (Kd contiguous), the K-major form the tcgen05 shared-memory descriptors
 *   read.  B200 counterpart of the reference's host-side weight format cast
 *   (torchair/npu_utils/npu_format_cast_via_cpu.cpp).
 *
 * tab_grouped_matmul_w8a8: x int8 [M, Kd]; packed weight; group_list int64 [E] (group_list_type 0 =
 *   cumulative row ends, 1 = row counts); expert e owns a contiguous row range.
 *   bias int32 [E, N] or NULL (the int8 mode's bias, grouped_matmul.py:258-262): acc += bias[e, n] in int32.
 *   out_dtype 3: y int32 [M, N] raw accumulators (scale, per_token_scale ignored);
 *   out_dtype 15 / 5: y = (float(acc) * per_token_scale[m]) * scale[e, n], scale fp32 [E, N],
 *   per_token_scale fp32 [M] (either may be NULL = 1).  Rows outside every group are left untouched.
 *   Requires Kd % 16 == 0.
 *   expected_rows_per_group (here and in the three entry points below): the rows a group is expected to hold, for the
 *   choice of kernel orientation and tile width on the host; 0 = unknown (M / E is assumed).  It is the first element of
 *   the operator's tuning_config, which the converter forwards to the IR attribute of that name without defining it
 *   (grouped_matmul.py:245,361; experiment_ops.h:3651); decision: expected rows per group.  With expert parallelism
 *   x is sized for the worst case, so M / E can be many times what arrives and the hint matters.  Any value gives
 *   correct results: the counts themselves are read on the device.
 *
 * tab_grouped_matmul_w8a8_scatter: the same GEMM with 16-bit output (out_dtype 15 or 5) whose row m is stored at the
 *   address row_dst[m] (device array of M addresses, 16-byte aligned rows of N elements) instead of y + m*N.  The
 *   addresses may lie in peer-mapped memory of another GPU: with tab_ep_return_plan this is the down projection of
 *   npu_grouped_matmul fused with the row return of npu_moe_distribute_combine (moe_distribute_combine.py:4-60),
 *   each tile leaving over NVLink as its epilogue finishes.  Rows outside every group, and rows whose table entry
 *   is 0, are not stored.  N % 8 == 0.
 *
 * tab_grouped_matmul_swiglu_quant: gate_up GEMM with the DequantSwigluQuant epilogue fused
 *   (grouped_matmul.py:210-365 followed by npu_dequant_swiglu_quant.py:5-64; the reference's own fused
 *   form is converter grouped_matmul_swiglu_quant_v2.py:86-166).  packed weight [E, 2*I, Kd];
 *   weight_scale fp32 [E, 2*I]; x_scale fp32 [M]; yq int8 [M, I]; y_scale fp32 [M]; rows outside every
 *   group are left untouched.  Workspace holds the fp32 SwiGLU values between the two phases.
 *
 * tab_grouped_matmul_finalize_routing: the down GEMM and the combine as one call (converter
 *   grouped_matmul_finalize_routing.py:57-133 -> GroupedMatmulFinalizeRouting, fusion_ops.h:640-725), int8 x and
 *   int8 weight only.  y fp32 [output_bs, N] = 0; rows [shared_input_offset, +shared_rows) = shared_input_weight *
 *   shared_input (bf16 [shared_rows, N], NULL to skip); then for every row m inside a group e:
 *   y[row_index[m]] += logit[m] * ((float(acc[m]) * per_token_scale[m]) * scale[e] + bias[e]),
 *   scale fp32 [E, N], bias bf16 [E, N], logit fp32 [M], per_token_scale fp32 [M] (each NULL = neutral),
 *   row_index int32 or int64 [M] (row_index_dtype 3 or 4; entries outside [0, output_bs) add nothing).
 *   The additions into one output row are 16-byte L2 reductions in no fixed order.  Requires N % 4 == 0;
 *   the workspace holds the int32 accumulators.
 *
 * tab_gmm_status: host-side; copies the device status word of the GEMM launches on this device
 *   (0 = fine, otherwise the code of the first bounded wait that gave up) after synchronising `stream`.  The word is
 *   sticky; tab_gmm_status_reset (host-side, synchronises `stream`) clears it.  Every wait inside the kernels is
 *   bounded (TAB_GMM_WAIT_MS in the environment, read once; default 2000 ms): on expiry the CTA records its code,
 *   drains its copies, frees its tensor memory and returns with its tiles unwritten, so callers that need to know
 *   poll this word where they synchronise anyway.
 * ------------------------------------------------------------------------------------------------- */
TAB_API int tab_prepack_weight_i8(const int8_t* weight, int64_t E, int64_t Kd, int64_t N, int8_t* packed,
                          tab_stream_t stream);
TAB_API int tab_grouped_matmul_w8a8(const int8_t* x, const int8_t* packed_weight, const float* scale,
                            const float* per_token_scale, const int32_t* bias, const int64_t* group_list, int group_list_type,
                            int64_t M, int64_t Kd, int64_t N, int64_t E, int out_dtype, void* y,
                            int64_t expected_rows_per_group, tab_stream_t stream);
TAB_API int tab_grouped_matmul_w8a8_scatter(const int8_t* x, const int8_t* packed_weight, const float* scale,
                                    const float* per_token_scale, const int64_t* group_list, int group_list_type,
                                    int64_t M, int64_t Kd, int64_t N, int64_t E, int out_dtype, const uint64_t* row_dst,
                                    int64_t expected_rows_per_group, tab_stream_t stream);
TAB_API int tab_grouped_matmul_swiglu_quant_workspace_bytes(int64_t M, int64_t I, size_t* bytes);
TAB_API int tab_grouped_matmul_swiglu_quant(const int8_t* x, const int8_t* packed_weight, const float* weight_scale,
                                    const float* x_scale, const int64_t* group_list, int group_list_type,
                                    int64_t M, int64_t Kd, int64_t I, int64_t E, int activate_left,
                                    int8_t* yq, float* y_scale, void* workspace, size_t workspace_bytes,
                                    int64_t expected_rows_per_group, tab_stream_t stream);
TAB_API int tab_grouped_matmul_finalize_routing_workspace_bytes(int64_t M, int64_t N, size_t* bytes);
TAB_API int tab_grouped_matmul_finalize_routing(const int8_t* x, const int8_t* packed_weight, const float* scale,
                                        const void* bias, const float* per_token_scale, const int64_t* group_list,
                                        int group_list_type, int64_t M, int64_t Kd, int64_t N, int64_t E,
                                        const void* shared_input, int64_t shared_rows, float shared_input_weight,
                                        int64_t shared_input_offset, const float* logit, const void* row_index,
                                        int row_index_dtype, int64_t output_bs, float* y, void* workspace,
                                        size_t workspace_bytes, int64_t expected_rows_per_group, tab_stream_t stream);
TAB_API int tab_gmm_status(int* status_host, tab_stream_t stream);
TAB_API int tab_gmm_status_reset(tab_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TAB_API_H_ */
