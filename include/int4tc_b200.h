/*
 * int4tc_b200 -- C ABI of the B200 (sm_100a) W4A4 int4 x int4 library.
 *
 * Every entry point takes raw device pointers, sizes, a CUDA device ordinal and a
 * CUDA stream handle (a `cudaStream_t` passed as `void*`; NULL = the legacy default
 * stream).  Nothing here depends on PyTorch.  Work is enqueued on `stream` and the
 * call returns without synchronising unless stated otherwise.
 *
 * Return value: 0 on success; a negative I4TC_E* code for a rejected argument; a
 * positive value is a `cudaError_t` raised by the runtime.  `i4tc_last_error()`
 * returns a human-readable message for the calling thread's last failure.
 *
 * Each declaration cites the reference interface it replaces, as
 * `file:line` inside the reference project (gkswns0531/fp8_inference_toolkit).
 *
 * Data formats (identical to the reference's):
 *   packed int4   : two's-complement nibbles, element 2i in the low nibble of byte i
 *                   (int4_native_tc/csrc/int4_quant.cu:49-51)
 *   row-major     : codes [R, K/2] u8, scale [R] f32               (per token / per channel)
 *   group-major   : codes [G, R, gs/2] u8, scale [G, R] f32, G=K/gs (int4_quant.cu:651-653)
 */
#ifndef INT4TC_B200_H_
#define INT4TC_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ---------------------------------------------------------- */
#define I4TC_OK 0
#define I4TC_EINVAL (-1)      /* bad shape / size / flag                         */
#define I4TC_EALIGN (-2)      /* pointer or stride not aligned as required       */
#define I4TC_EUNSUPPORTED (-3)/* combination not implemented                     */
#define I4TC_EDEVICE (-4)     /* device is not compute capability 10.x           */
#define I4TC_EKERNEL (-5)     /* a kernel reported a bounded-wait timeout        */
#define I4TC_EWORKSPACE (-6)  /* the split-K workspace could not be grown        */

/* element types of floating-point inputs / outputs */
#define I4TC_BF16 0
#define I4TC_FP16 1
#define I4TC_FP32 2
#define I4TC_INT32 3

/* scale conventions (int4_quant.cu:142 vs :267) */
#define I4TC_ROLE_ACTIVATION 0 /* scale = max(absmax/7, 1/(7*512))              */
#define I4TC_ROLE_WEIGHT 1     /* scale = absmax/7, or 1.0 for an all-zero slice */

int i4tc_version(void);
const char* i4tc_last_error(void);

/* Number of SMs of `device` (cached); negative on error. */
int i4tc_sm_count(int device);

/* Test / tuning hook: force the GEMM tile width (64, 128, 256; 0 = automatic) and the operand
 * orientation (1 = weights on the 128-row side of the MMA, 0 = activations, -1 = automatic).
 * Process-wide.  Results do not depend on it. */
int i4tc_set_tuning(int tile_n, int swap);

/* Test / tuning hook for the small-M paths with scaled outputs (9..128 tokens): number of K ranges that
 * different thread blocks handle before a fixed-order reduction (0 = automatic, 1 = never split, 2..8 = forced;
 * per-channel results do not depend on it, per-group results only in the order fp32 terms are added).  The
 * partial sums live in a workspace owned by the library, see i4tc_reserve_workspace. */
int i4tc_set_split_k(int splits);

/* The split-K workspace.  The small-M GEMMs (9..128 tokens, scaled outputs) may cut K into up to 8 ranges whose
 * fp32 partial sums (splits * M * N * 4 bytes, at most 4 KiB per output column) go to a buffer that the library
 * owns, one per (device, stream): calls on different streams never share it.  A buffer that a call has used is never
 * freed or moved afterwards -- a launch in flight or a CUDA graph captured earlier may still hold its address -- so
 * when a stream needs more than it has, a larger buffer is allocated beside the old one (geometric growth, 16 MiB
 * minimum).  That allocation is a cudaMalloc inside the GEMM call: to keep it out of a stream capture or a
 * latency-critical loop, reserve the largest size beforehand with i4tc_reserve_workspace (any thread, outside
 * capture; 100 MiB covers N = 24576).  If the allocation fails the GEMM call returns I4TC_EWORKSPACE and launches
 * nothing.  i4tc_workspace_bytes reports the current size for a stream; i4tc_release_workspaces synchronises the
 * device and frees every buffer of it (only when no captured graph that used them will be replayed).  Two replays
 * of graphs captured on one stream that run concurrently on different streams share that stream's buffer and race.
 * No reference counterpart. */
int i4tc_reserve_workspace(int device, void* stream, int64_t bytes);
int64_t i4tc_workspace_bytes(int device, void* stream);
int i4tc_release_workspaces(int device);

/* Test / tuning hook for large dense problems: whether pairs of thread blocks on two SMs share 256 x 256
 * tiles (-1 = automatic, 0 = never, 1 = whenever the problem allows it: 256-wide tiles, activations on the
 * row side, scaled outputs).  Process-wide.  Results do not depend on it.  No reference counterpart. */
int i4tc_set_cta_pairs(int mode);

/* Test / tuning hook: number of epilogue warps per thread block of the tensor-core GEMM (0 = automatic, 8 or 16;
 * 64-column tiles always use 8).  Process-wide.  Results do not depend on it.  No reference counterpart. */
int i4tc_set_epilogue_warps(int warps);

/* Test / tuning hook: which kernel serves a linear with few tokens (0 = automatic: the CUDA-core weight-streaming
 * kernel for one or two tokens, the register-fed tensor-core one up to 32 (16 with per-channel scales), the tile kernel
 * beyond; 1 = the CUDA-core kernel
 * where it applies, else the tile kernel; 2 = the register-fed kernel wherever it applies (1..32 tokens); 3 = always
 * the tile kernel).  Process-wide.  Per-channel results do not depend on it; per-group results differ only in the
 * order in which fp32 partial sums over K ranges are added.  No reference counterpart. */
int i4tc_set_small_m_path(int path);

/* ---- quantise + pack ------------------------------------------------------- */

/* Per-row symmetric int4 quantise + pack, one pass over the input.
 * Replaces dynamic_int4_quant (int4_native_tc/csrc/int4_quant.cu:201, kernel :100)
 * and static_int4_weight_quant (int4_quant.cu:289, kernel :240); `role` selects
 * between their scale conventions.  x: [rows, K] of `dtype`, row stride `ldx`
 * elements; packed: [rows, K/2]; scale: [rows].  K must be even. */
int i4tc_quant_rowwise(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                       uint8_t* packed, float* scale, int role, int device, void* stream);

/* Per-(row, group) symmetric int4 quantise + pack with group-major outputs.
 * Replaces dynamic_int4_quant_grouped (int4_quant.cu:806, kernel :759) and
 * static_int4_weight_quant_grouped (int4_quant.cu:712, kernel :665).
 * packed: [K/gs, rows, gs/2]; scale: [K/gs, rows].  gs in {32,64,128,256}, K % gs == 0. */
int i4tc_quant_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                       int64_t group_size, uint8_t* packed, float* scale, int role,
                       int device, void* stream);

/* Quantise + pack with caller-supplied divisors: q = clamp(rint(x / scale), -8, 7).
 * group_size == 0: scale [rows], packed row-major; otherwise scale [K/gs, rows] and
 * packed group-major.  No reference op has this signature; it is the "identical
 * scales" form under which codes are compared bit for bit with the CPU oracle
 * (arithmetic of benchmark/benchmark_w4a8fp8.py:200-204). */
int i4tc_quant_with_scales(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                           int64_t group_size, const float* scale, uint8_t* packed,
                           int device, void* stream);

/* Per-(row, group) symmetric int4 quantise + pack whose range is the group's absmax * clip_ratio:
 *   s = absmax * clip_ratio / 7;  q = clamp(rint(x / s), -8, 7);  scale = max(s, 1/(7*512)).
 * Replaces dynamic_int4_quant_clipped_grouped (int4_quant.cu:906, kernel :857).  x bf16 or fp16;
 * gs in {64,128,256}; clip_ratio in (0, 1]; packed [K/gs, rows, gs/2] (4-byte aligned); scale [K/gs, rows]. */
int i4tc_quant_clipped_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                               int64_t group_size, double clip_ratio, uint8_t* packed, float* scale,
                               int device, void* stream);

/* Per-(row, group) asymmetric int4 quantise + pack:
 *   v = x (or x / smooth_scale[k] when smooth_scale != NULL: [K], same dtype as x);
 *   c = clamp(v, -t, t) with t = max|v| * clip_ratio;  s = max((max c - min c) / 15, 1/(7*512));
 *   azp = clamp(rint(-min c / s), 0, 15);  u = clamp(rint(c / s + azp), 0, 15);
 *   stored nibble = u - 8 (so the GEMM sees signed codes);  azp_adj = 8 - azp.
 * Replaces dynamic_int4_quant_asymmetric_grouped (int4_quant.cu:1262, kernel :1189; clip_ratio = 1,
 * smooth_scale = NULL) and dynamic_int4_quant_asymmetric_clipped_grouped (int4_quant.cu:1433, kernel :1324).
 * Outputs: packed [K/gs, rows, gs/2] (4-byte aligned), scale [K/gs, rows], azp_adj [K/gs, rows]. */
int i4tc_quant_asymmetric_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                                  int64_t group_size, double clip_ratio, const void* smooth_scale,
                                  uint8_t* packed, float* scale, float* azp_adj, int device, void* stream);

/* out[r] = float(sum of the signed 4-bit codes of packed row r), r < rows, each row group_size / 2 bytes:
 * on group-major weights [G, N, gs/2] (rows = G * N) this is the w_col_sum [G, N] operand of the zero-point
 * GEMM.  The reference computes it in torch when weights are prepared (int4_native_tc/profile_layer.py:96-119). */
int i4tc_weight_group_sums(const uint8_t* b_packed, int64_t rows, int64_t group_size, float* out,
                           int device, void* stream);

/* packed [rows, K/2] -> int8 [rows, K] with sign extension.
 * Replaces unpack_int4_to_int8 (int4_quant.cu:593, kernel :553). */
int i4tc_unpack_int4_to_int8(const uint8_t* packed, int64_t rows, int64_t K, int8_t* out,
                             int device, void* stream);

/* ---- dense W4A4 GEMM ------------------------------------------------------- */

/* C[m,n] = sum_k A[m,k] * B[n,k], int32 out [M,N] (row stride N).
 * a: [M, K/2], b: [N, K/2] row-major packed.  K % 64 == 0.
 * Replaces cutlass_int4_gemm (int4_native_tc/csrc/int4_gemm.cu:779). */
int i4tc_gemm_int32(const uint8_t* a, const uint8_t* b, int32_t* c, int64_t M, int64_t N,
                    int64_t K, int device, void* stream);

/* out[m,n] = cast((float(acc) * scale_b[n]) * scale_a[m]); out_dtype BF16 or FP16, [M,N].
 * Replaces cutlass_int4_scaled_mm (int4_gemm.cu:831; epilogue :137-150). */
int i4tc_gemm_scaled(const uint8_t* a, const uint8_t* b, const float* scale_a,
                     const float* scale_b, void* out, int out_dtype, int64_t M, int64_t N,
                     int64_t K, int device, void* stream);

/* W4A8: int8 activations x int4 weights held as int8 (the output of i4tc_unpack_int4_to_int8), both [rows, K]
 * row-major; out[m,n] = cast((int32 acc * scale_b[n]) * scale_a[m]).  Replaces cutlass_w4a8_scaled_mm
 * (int4_native_tc/csrc/int4_gemm.cu:874-899, kernel instantiation :284-378).  K must be a multiple of 32 (as
 * int4_gemm.cu:885); a and b 16-byte aligned.  The operands go by TMA straight into the swizzled int8 stages of the
 * tensor-core kernel (nothing is converted). */
int i4tc_gemm_w4a8_scaled(const int8_t* a, const int8_t* b, const float* scale_a, const float* scale_b,
                          void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int device, void* stream);

/* Per-token symmetric int8 quantise: q int8 [rows, K], scale fp32 [rows] = max(absmax / 127, 1 / (127 * 512)).
 * Replaces dynamic_int8_quant (int4_native_tc/csrc/int4_quant.cu:432-537). */
int i4tc_quant_rowwise_int8(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int8_t* q,
                            float* scale, int device, void* stream);

/* Per-group-128 fused linear:
 *   out[m,n] = bf16( sum_g (float(acc_g[m,n]) * scale_a[g,m]) * scale_b[g,n] ), g ascending.
 * a: [G, M, 64], b: [G, N, 64] group-major packed; scale_a [G,M]; scale_b [G,N]; out bf16 [M,N].
 * Replaces cutlass_int4_fused_grouped_gemm and its same-contract aliases _v5/_v7/_v8/_v9
 * (int4_gemm.cu:4231, 3751, 4073, 4007, 3932) and cutlass_int4_scaled_mm_grouped (:929).
 * `group_size` must be 128 (as int4_gemm.cu:4243). */
int i4tc_gemm_grouped(const uint8_t* a, const uint8_t* b, const float* scale_a,
                      const float* scale_b, void* out, int64_t M, int64_t N,
                      int64_t group_size, int64_t num_groups, int device, void* stream);

/* Per-group-128 fused linear for asymmetrically quantised activations:
 *   out[m,n] = bf16( sum_g scale_a[g,m] * scale_b[g,n] * (acc_g[m,n] + azp_adj[g,m] * w_col_sum[g,n]) ).
 * Replaces cutlass_int4_fused_grouped_gemm_azp and its aliases _v5_azp / _v7_azp (int4_gemm.cu:4298, 3838,
 * 4149; epilogue term :1851-1858) and cutlass_int4_scaled_mm_azp_grouped (:994).  Same operands as
 * i4tc_gemm_grouped plus azp_adj [G, M] and w_col_sum [G, N] (fp32).  The term is added to each group's integer
 * sum inside the epilogue of the tensor-core kernel, before the scales, in the reference's order
 * ((acc + azp * wcs) * sx, then the fused multiply-add by sw); no workspace, no second kernel. */
int i4tc_gemm_grouped_azp(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                          const float* azp_adj, const float* w_col_sum, void* out, int64_t M, int64_t N,
                          int64_t group_size, int64_t num_groups, int device, void* stream);

/* int32 partial sums of every group, out [G, M, N]: the integer accumulators that the fused
 * kernel drains.  No reference op exposes them; used to check the integer path bit for bit. */
int i4tc_gemm_grouped_int32(const uint8_t* a, const uint8_t* b, int32_t* out, int64_t M,
                            int64_t N, int64_t num_groups, int device, void* stream);

/* ---- MoE (no counterpart in the reference; composition of the grouped ops) -- */

/* Stable counting sort of the T*top_k (token, slot) pairs by expert id.
 * expert_ids: [num_pairs] int32 in [0, E); ids outside that range are left out.
 * Outputs: sorted_pairs [num_pairs] int32 (pair index = token*top_k + slot, ascending inside an
 * expert; the entries past expert_offsets[E], which left-out pairs would have filled, are set to -1),
 * inv_pairs [num_pairs] (sorted position of each pair, -1 if left out; may be NULL),
 * expert_offsets [E+1] int32.  E <= 256.  `scratch` is caller-provided device memory of at least
 * i4tc_moe_sort_scratch_bytes(num_pairs, E) bytes that the sort uses for per-chunk histograms. */
int64_t i4tc_moe_sort_scratch_bytes(int64_t num_pairs, int64_t num_experts);
int i4tc_moe_sort(const int32_t* expert_ids, int64_t num_pairs, int64_t num_experts,
                  int32_t* sorted_pairs, int32_t* inv_pairs, int32_t* expert_offsets,
                  void* scratch, int64_t scratch_bytes, int device, void* stream);

/* The same sort for callers that cannot allocate device memory when they call it -- for example an
 * inference server whose own pool already owns all free HBM, or a latency-critical loop that must
 * avoid cudaMalloc/cudaFree because they synchronise the device.  It has no counterpart in the
 * reference.  The scratch is a fixed 64 KiB array inside the library (held by every GPU that loads
 * it, until exit), so the limit is ceil(num_pairs / 1024) * num_experts <= 16384 entries
 * (i4tc_moe_sort_noalloc_max_scratch_ints()); larger problems are rejected with I4TC_EINVAL and
 * should use i4tc_moe_sort.  The call itself allocates nothing: no cudaMalloc, no cudaFree, no library
 * allocator.  One thing happens only once per device: the first use there looks up the array's device
 * address (cudaGetSymbolAddress), and if nothing of this library's MoE code ran on that device before, the
 * CUDA runtime loads the code module at that moment -- with lazy module loading that is when the driver
 * sets aside the 64 KiB array and the kernels' code, which does need free device memory.  So do that first
 * use at start-up, while memory is still free and before any stream capture: call
 * i4tc_moe_sort_noalloc_prepare(device) (launches nothing) or make one call with num_pairs = 0.  All calls
 * share the one array, which keeps whatever the last call left in it (no entry has to start at
 * zero: each call overwrites what it reads), so two calls that overlap on the GPU -- different
 * streams, or different threads -- race; keep them ordered.  Outputs are identical to i4tc_moe_sort. */
int64_t i4tc_moe_sort_noalloc_max_scratch_ints(void);
int i4tc_moe_sort_noalloc_prepare(int device);
int i4tc_moe_sort_noalloc(const int32_t* expert_ids, int64_t num_pairs, int64_t num_experts,
                          int32_t* sorted_pairs, int32_t* inv_pairs, int32_t* expert_offsets,
                          int device, void* stream);

/* Gather rows x[sorted_pairs[i] / top_k] and grouped-quantise them (gs=128, activation
 * role) straight into expert-sorted group-major layout: packed [K/128, P, 64], scale [K/128, P].
 * x has num_tokens rows; a pair index outside [0, num_tokens * top_k) (the -1 entries the sort leaves for
 * left-out pairs) reads nothing and is quantised as a row of zeros. */
int i4tc_moe_gather_quant(const void* x, int dtype, int64_t num_tokens, int64_t K, int64_t ldx,
                          const int32_t* sorted_pairs, int64_t num_pairs, int64_t top_k,
                          uint8_t* packed, float* scale, int device, void* stream);

/* The same result from rows that were quantised once per token (i4tc_quant_grouped over x, group size 128:
 * tok_packed [G, T, 64], tok_scale [G, T]) -- the quantiser works on whole rows, so quantising a token once and
 * copying its 68 bytes per group to every (token, slot) pair gives the codes and scales of quantising after the
 * gather, with top_k times less arithmetic.  Destination: group-major packed [G, P, 64] / scale [G, P] (row_map NULL),
 * or, for the expert-parallel exchange, rows of row_bytes = 68 G bytes at row row_map[i] of a block buffer (`packed`,
 * or with peer_bases the destination ranks' buffers as in i4tc_moe_ep_dispatch_quant).  Pair indices that are negative
 * or name no token copy nothing. */
int i4tc_moe_gather_packed(const uint8_t* tok_packed, const float* tok_scale, int64_t num_tokens,
                           int64_t num_groups, const int32_t* pairs, int64_t num_pairs, int64_t top_k,
                           uint8_t* packed, float* scale, const int32_t* row_map, int64_t row_bytes,
                           const uint64_t* peer_bases, int64_t cap, int64_t my_rank, int device, void* stream);

/* Grouped-tile W4A4 GEMM over expert-sorted rows:
 *   for rows r in [expert_offsets[e], expert_offsets[e+1]):  out[r, :] = linear_grouped(a[:, r, :], W_e)
 * a: [G, P, 64], scale_a [G, P]; b: [E, G, N, 64], scale_b [E, G, N]; out bf16 [P, N].
 * `expert_offsets` is read on the device (no host synchronisation). */
int i4tc_moe_grouped_gemm(const uint8_t* a, const float* scale_a, const uint8_t* b,
                          const float* scale_b, const int32_t* expert_offsets, void* out,
                          int64_t num_pairs, int64_t N, int64_t num_groups,
                          int64_t num_experts, int device, void* stream);
/* The same GEMM with every output row written to its own address (out_rows [num_pairs], device array of 16-byte aligned
 * addresses, N bf16 values each) instead of out + row * N: the expert-parallel layer lets the down projection write
 * straight into the return buffers of the ranks the rows came from (i4tc_moe_ep_return_rows builds the table; rows in
 * another GPU's memory are reached with plain stores over NVLink).  N must be a multiple of 8.  No reference counterpart. */
int i4tc_moe_grouped_gemm_rows(const uint8_t* a, const float* scale_a, const uint8_t* b,
                               const float* scale_b, const int32_t* expert_offsets, const uint64_t* out_rows,
                               int64_t num_pairs, int64_t N, int64_t num_groups, int64_t num_experts,
                               int device, void* stream);

/* RMSNorm fused in front of the grouped quantiser: for every row of x (bf16 [rows, K], row stride ldx)
 *   y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * norm_weight[k]),  then y is quantised like i4tc_quant_grouped
 * (activation role) -> packed [K/group_size, rows, group_size/2], scale [K/group_size, rows].
 * No reference counterpart: the reference quantises the output of a separate normalisation; its report names
 * this fusion as the follow-up (docs/native_int4_tc_implementation_report.md:515-562). */
int i4tc_rmsnorm_quant_grouped(const void* x, int64_t rows, int64_t K, int64_t ldx, const void* norm_weight,
                               float eps, int64_t group_size, uint8_t* packed, float* scale, int device,
                               void* stream);

/* SwiGLU + grouped re-quantise: h bf16 [P, 2I] laid out [gate | up] ->
 * act = bf16(silu(gate) * up) -> packed [I/128, P, 64], scale [I/128, P]. */
int i4tc_moe_silu_mul_quant(const void* h, int64_t P, int64_t I, uint8_t* packed, float* scale,
                            int device, void* stream);

/* ---- expert parallelism with fixed-capacity exchange buffers (no counterpart in the reference) ----
 *
 * One layer on a rank: i4tc_moe_sort (by global expert id) -> i4tc_moe_ep_plan -> i4tc_moe_ep_dispatch_quant ->
 * all-to-all of the send buffer (equal blocks, so no split sizes ever leave the device) -> i4tc_moe_ep_unpack ->
 * i4tc_moe_grouped_gemm / i4tc_moe_silu_mul_quant_rows / i4tc_moe_grouped_gemm -> i4tc_moe_ep_pack_return ->
 * all-to-all back -> i4tc_moe_combine with ret_row as the row index.
 *
 * Buffers.  send / recv: `world` blocks of (1 + cap) rows of row_bytes = (H / 128) * 68 bytes: a header row, then up
 * to cap token rows (64 bytes of codes and one fp32 scale per group of 128), in the source's sorted order.
 * slot [num_pairs]: buffer row of each sorted position (-1: beyond the capacity).  ret_row [num_pairs]: for every
 * (token, slot) pair the row of the returned [world * cap, H] buffer that holds its expert output (-1: none).
 * overflow: device word, bit 0 set when a destination would have received more than cap rows -- the layer's result
 * is then incomplete and the caller repeats the step with exact split sizes; nothing is ever read or written out of
 * range.  meta: int32 scratch of i4tc_moe_ep_meta_ints(world, e_loc) entries.  rows_dev: device int32, rows received.
 *
 * Peer destinations.  Where the ranks' receive and return buffers are mapped into the address space of every other rank
 * (symmetric memory over NVLink), peer_bases [world] (device array of addresses: the receive buffer of rank d for the
 * plan and dispatch calls, the return buffer [num_pairs, H] of rank s for the pack_return call) makes the kernels store
 * rows straight into the buffer of the destination -- block `my_rank` of the receive buffer of d, row (start + j) of the
 * return buffer of s, i.e. the sorted order of the source, so that the source combines with inv_pairs as on one GPU -- and
 * no all-to-all is needed; the ranks order their accesses with i4tc_peer_signal / i4tc_peer_wait.  With
 * peer_bases = NULL everything goes to the local send buffers as described above. */
int i4tc_moe_ep_plan(const int32_t* expert_offsets, const int32_t* sorted_pairs, int64_t num_pairs,
                     int64_t num_experts, int64_t world, int64_t cap, int64_t row_bytes, void* send_buf,
                     int32_t* slot, int32_t* ret_row, unsigned int* overflow, const uint64_t* peer_bases,
                     int64_t my_rank, int device, void* stream);
int i4tc_moe_ep_dispatch_quant(const void* x, int64_t num_tokens, int64_t K, int64_t ldx,
                               const int32_t* sorted_pairs, int64_t num_pairs, int64_t top_k,
                               const int32_t* slot, void* send_buf, int64_t row_bytes,
                               const uint64_t* peer_bases, int64_t cap, int64_t my_rank, int device, void* stream);
/* flag_addrs [world] (device array): address, in the flag array of every rank, of the slot that belongs to this rank.
 * Once all earlier work of `stream` is done the slot receives `epoch` (system-scope release).  i4tc_peer_wait makes
 * `stream` wait until all `world` slots of the local array `flags` have reached `epoch`; after two seconds it gives
 * up, sets bit 1 of the status word (i4tc_check_status) and lets the stream continue.  Epochs grow by one per
 * exchange; waiting and signalling kernels of different ranks run on different GPUs. */
int i4tc_peer_signal(const uint64_t* flag_addrs, int64_t world, uint32_t epoch, int device, void* stream);
int i4tc_peer_wait(const uint32_t* flags, int64_t world, uint32_t epoch, int device, void* stream);
/* The same pair with the epoch held in device memory (`counter`, one uint32 per layer object), for layers that are
 * replayed as a CUDA graph: a signal with bump != 0 first adds one to the counter, every other call uses its current
 * value.  One exchange layer = signal(bump = 1), wait, ..., signal(bump = 0) on a second flag array, wait.
 * No reference counterpart. */
int i4tc_peer_signal_counter(const uint64_t* flag_addrs, int64_t world, uint32_t* counter, int bump, int device,
                             void* stream);
int i4tc_peer_wait_counter(const uint32_t* flags, int64_t world, const uint32_t* counter, int device, void* stream);
int64_t i4tc_moe_ep_meta_ints(int64_t world, int64_t e_loc);
/* a_packed [G, world * cap, 64], a_scale [G, world * cap]: received rows in expert-sorted order (rows past *rows_dev
 * are not written); expert_offsets_loc [e_loc + 1]; pos_of [world * cap]: sorted position of received row (s, j). */
int i4tc_moe_ep_unpack(const void* recv_buf, int64_t world, int64_t e_loc, int64_t cap, int64_t row_bytes,
                       int64_t num_groups, uint8_t* a_packed, float* a_scale, int32_t* expert_offsets_loc,
                       int32_t* pos_of, int32_t* meta, int32_t* rows_dev, int device, void* stream);
/* i4tc_moe_silu_mul_quant over the first *rows_dev of max_rows rows (the count stays on the device). */
int i4tc_moe_silu_mul_quant_rows(const void* h, int64_t max_rows, const int32_t* rows_dev, int64_t I,
                                 uint8_t* packed, float* scale, int device, void* stream);
/* ret_send[row, :] = y[pos_of[row], :] for the `rows` = world * cap buffer rows (bf16 [.., H]); rows without a
 * received token (pos_of < 0) are left as they are. */
int i4tc_moe_ep_pack_return(const void* y, const int32_t* pos_of, int64_t rows, int64_t H, void* ret_send,
                            const uint64_t* peer_bases, const int32_t* meta, int64_t world, int64_t e_loc,
                            int64_t cap, int device, void* stream);
/* out_rows [world * cap] (device): for every expert-sorted row of this rank the address of its place in the return
 * buffer of the rank it came from (peer_bases, meta, geometry as for i4tc_moe_ep_pack_return), for
 * i4tc_moe_grouped_gemm_rows; entries of positions that hold no row are left alone.  No reference counterpart. */
int i4tc_moe_ep_return_rows(const int32_t* pos_of, int64_t rows, int64_t H, const uint64_t* peer_bases,
                            const int32_t* meta, int64_t world, int64_t e_loc, int64_t cap, uint64_t* out_rows,
                            int device, void* stream);

/* out[t, :] = bf16( sum_j w[t, j] * y[inv_pairs[t*top_k + j], :] ), j ascending, fp32 sum.
 * y bf16 [P, H]; inv_pairs[pair] = sorted position of that pair. */
int i4tc_moe_combine(const void* y, const int32_t* inv_pairs, const float* w, int64_t T,
                     int64_t top_k, int64_t H, void* out, int device, void* stream);

/* Polls the device-side status word written by bounded waits; 0 if no kernel timed out since
 * the last call, else I4TC_EKERNEL.  Synchronises `stream`. */
int i4tc_check_status(int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INT4TC_B200_H_ */
