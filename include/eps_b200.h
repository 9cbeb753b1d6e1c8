/*
 * eps_b200 — C ABI of the B200 (sm_100a) FP8 MoE expert-layer kernels.
 *
 * This is the boundary a binding of the reference (meituan-longcat/eps) would
 * call instead of its own CUDA: plain pointers and sizes, no torch types.
 * Every pointer is a DEVICE pointer unless its comment says "host".  `stream`
 * is a cudaStream_t passed as void*.  Every function returns EPSB_OK (0) or an
 * EPSB_ERR_* code; epsb_last_error() then returns a message for the calling
 * thread.  Launches are asynchronous on `stream`; nothing here synchronises
 * unless stated.  No function allocates device memory unless stated.
 *
 * Citations "ref: path:line" are paths inside the reference repository and
 * name the interface each entry point replaces.
 *
 * Index conventions (identical to the reference): T local tokens, k = top-k,
 * E routed FFN experts, W expert-parallel world size, EL = E/W local experts,
 * S stages (S divides EL), R rows received by a rank, D expanded GEMM rows.
 * A negative expert id is a zero-computation (identity) expert.
 */
#ifndef EPS_B200_H_
#define EPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EPSB_OK 0
#define EPSB_ERR_INVALID 1  /* bad argument / unsupported shape (reference: std::runtime_error) */
#define EPSB_ERR_CUDA 2     /* a CUDA runtime/driver call failed */
#define EPSB_ERR_TIMEOUT 3  /* a bounded device-side wait gave up (word 0 of the GEMM's status buffer) */
#define EPSB_ERR_WORKSPACE 4 /* workspace too small */

const char* epsb_last_error(void);
int epsb_version(void);

/* ----------------------------------------------------------------------------
 * Quantisation.  ref: src/quant/fp8.cuh:43-72, src/quant/fp8.cu:247-382
 * (per_token_group_quant_fp8<T,Params>, group_size 128).
 *
 * x: [rows, cols] bf16 row-major, cols % 128 == 0.
 * q: [rows, cols] e4m3 codes.  scales: [rows, cols/128] fp32 row-major.
 * div_mode 1: scale = div.full.f32(amax, 448), the instruction the reference kernel uses (fp8.cu:272-275);
 *             bit-identical to that kernel (on B200 it equals amax * fl(1/448) for every input).
 * div_mode 0: scale = amax/448 with IEEE division (differs from mode 1 by 1 ulp on ~59 % of scales).
 * -------------------------------------------------------------------------- */
int epsb_quant_1x128(const void* x, int64_t rows, int64_t cols, void* q, float* scales, int div_mode, void* stream);

/* Ragged form (PerTokenGroupQuantFP8Params, fp8.cuh:43-57): only rows
 * [exclusive_sum[0], exclusive_sum[num_experts]) are processed; the bounds are
 * read on the device.  max_rows bounds the grid (reference: num_tokens_hint). */
int epsb_quant_1x128_ragged(const void* x, const int32_t* exclusive_sum, int num_experts, int64_t cols, void* q,
                            float* scales, int64_t max_rows, int div_mode, void* stream);

/* Inverse (ref: fp8.cu:299-330): x = bf16(float(code) * scale). */
int epsb_dequant_1x128(const void* q, const float* scales, int64_t rows, int64_t cols, void* x, void* stream);

/* Weight quantisation: w [n_mats, n, k] bf16 -> codes [n_mats, n, k] and one
 * fp32 scale per 128x128 block, scales [n_mats, ceil(n/128), ceil(k/128)],
 * scale = amax/448 (IEEE).  The reference ships no block-scaled weight
 * quantiser; the slot it fills is GemmInterface::RunParams::weight_scales
 * (ref: src/scheduler/gemm_executor_interface.cuh:7-10).  k % 16 == 0. */
int epsb_quant_block128(const void* w, int64_t n_mats, int64_t n, int64_t k, void* q, float* scales, void* stream);

/* ----------------------------------------------------------------------------
 * Router: group-limited top-k over sigmoid scores; produces the expert_indices /
 * expert_scales the plans read.
 * ref: topk_sigmoid (src/utils/topk_sigmoid.cu:158-286, params
 *      src/utils/topk_sigmoid.cuh:6-19), which the reference instantiates for
 *      num_experts 256 / 8 groups / topk 8 only and otherwise throws
 *      "Not supported num_experts: ...".
 * Here: num_experts a multiple of 32 up to 1024, num_expert_groups dividing it
 * (<= 32), topk <= 32.
 *   score = 1/(1+expf(-logit)); biased = score + bias[e] (bias may be NULL);
 *   group score = sum of the group's two largest biased scores; the topk_groups
 *   best groups stay; topk times the largest biased score among their experts;
 *   expert_scales = score * route_scale / (sum of the chosen scores), fp32.
 * Ties go to the lower id.  Outputs [num_tokens, topk] in selection order.
 * Ids >= num_ffn_experts are written as -1 - (id - num_ffn_experts), the
 * identity-expert convention of the scheduler (comm_expander_ver2.cu:70-71);
 * pass num_ffn_experts = num_experts for no mapping.
 * logits [num_tokens, num_experts] fp32, or bf16 when logits_are_bf16 != 0.
 * -------------------------------------------------------------------------- */
int epsb_router_topk_sigmoid(const void* logits, int logits_are_bf16, const float* bias, int num_tokens,
                             int num_experts, int num_expert_groups, int topk_groups, int topk, float route_scale,
                             int num_ffn_experts, int32_t* expert_indices, float* expert_scales, void* stream);

/* The same selection with a choice of score function.  EPSB_ROUTER_SOFTMAX (no counterpart in the reference, whose
 * router is sigmoid only): score = expf(logit - max) / sum over the token's experts; everything after the score
 * (bias, groups, top-k, renormalisation of the chosen scores to route_scale) as above. */
#define EPSB_ROUTER_SIGMOID 0
#define EPSB_ROUTER_SOFTMAX 1
int epsb_router_topk(int score_func, const void* logits, int logits_are_bf16, const float* bias, int num_tokens,
                     int num_experts, int num_expert_groups, int topk_groups, int topk, float route_scale,
                     int num_ffn_experts, int32_t* expert_indices, float* expert_scales, void* stream);

/* ----------------------------------------------------------------------------
 * RMS normalisation of bf16 rows (a caller of the path in a full model):
 *   out[r, c] = bf16( (x[r, c] * rsqrt(mean_c(x[r, :]^2) + eps)) * scale[c] ), fp32 arithmetic.
 * ref: rms_norm (src/utils/rms_norm.cu:103-140), torch op utils.rms_norm_op
 *      (src/utils/bindings/th_rms_norm.cu:13-35).  n must be even ("dim ... is
 *      not divisible by 2.", as the reference).  out, input [m, n] bf16, scale [n] bf16.
 * -------------------------------------------------------------------------- */
int epsb_rms_norm(void* out, const void* input, const void* scale, float eps, int64_t m, int64_t n, void* stream);

/* ----------------------------------------------------------------------------
 * EPS scheduler plans.  All emit index layouts bit-identical to the reference.
 *
 * max_cluster (no counterpart in the reference, whose plan kernels are single
 * CTAs): the plan kernels run as one thread-block cluster of 1, 2, 4 or 8 CTAs,
 * chosen per call from the item count; max_cluster caps that (0 = up to 8).  A
 * caller that runs a plan next to a kernel occupying almost every SM passes 1,
 * because a cluster only starts once all of its CTAs fit into one GPC.
 * -------------------------------------------------------------------------- */

/* Source-side plans, one launch.
 * ref: CommExpander::plan -> getExpandForCommPlanKernel_ver2
 *      (src/scheduler/comm_expander.cuh:63-85, comm_expander_ver2.cu:30-183);
 *      GlobalReducer::plan -> getGlobalReducePlanKernel_ver2
 *      (src/scheduler/global_reducer.cuh:72-100, global_reducer_ver2.cu:31-215);
 *      ZeroReducer::plan -> zeroReducePlanKernel (src/scheduler/zero_reducer.cu:11-32).
 * in : idx [T,k] int32, weights [T,k] fp32 (may be NULL -> zero_scale untouched)
 * out: send_map [T*W] (first send_incl[W*S-1] entries valid) = ep*T + src
 *      send_incl [W*S] inclusive row counts by (dest rank, stage of leading expert)
 *      glob_map [T*W]: [t*W+ep] -> row of the returned buffer, or T*W
 *      coll_incl [W*S] inclusive counts by (dest rank, stage of tailing expert)
 *      zero_scale [T] = sum of weights of the token's zero-computation slots
 * Any of glob_map/coll_incl (together) or zero_scale may be NULL to skip. */
int epsb_source_plans(const int32_t* idx, const float* weights, int T, int k, int E, int W, int S, int32_t* send_map,
                      int32_t* send_incl, int32_t* glob_map, int32_t* coll_incl, float* zero_scale, int max_cluster,
                      void* stream);

/* The zero-expert plan alone, for callers that learn the gate weights after the sends were planned (the reference
 * computes it in Scheduler::plan, after rendezvous): zero_scale[t] = sum of weights[t,j] over slots with idx[t,j] < 0,
 * in slot order.  ref: zeroReducePlanKernel (src/scheduler/zero_reducer.cu:11-32). */
int epsb_zero_plan(const int32_t* idx, const float* weights, int T, int k, float* zero_scale, void* stream);

/* Receive plan from the all-gathered send plans.
 * ref: AlltoallRunner::plan -> getRecvPlan<512>
 *      (src/communication/alltoall_runner.cuh:79-103, alltoall_runner.cu:60-101).
 * gathered [W][W*S]: row d = rank d's inclusive plan.  recv_incl [W*S],
 * remote_offset [W*S] (where my stage block lands at each peer).
 * total_rows: optional pointer (device or host-mapped) that receives R. */
int epsb_recv_plan(const int32_t* gathered, int my_rank, int W, int S, int32_t* recv_incl, int32_t* remote_offset,
                   int32_t* total_rows, void* stream);

/* Expert-side plans, one launch.
 * ref: GemmExpander::plan -> getExpandForGemmPlanKernel_ver2
 *      (src/scheduler/gemm_expander.cuh:72-103, gemm_expander_ver2.cu:31-186);
 *      LocalReducer::plan -> getLocalReducePlanKernel_ver2{,_decode}
 *      (src/scheduler/local_reducer.cuh:78-114, local_reducer_ver2.cu:25-484).
 * in : ridx [R,k] expert ids of received rows; recv_incl [W*S] (R is read from
 *      recv_incl[W*S-1] on the device); local experts [lo,hi); max_rows bounds R.
 * out: excl [EL+1]; gemm_map [max_rows*k] (first excl[EL] valid) = row*k+slot
 *      inv_gemm [max_rows*k]: [row*k+slot] -> GEMM row or R*k (scratch the
 *      caller provides; also useful to callers that fuse the gather)
 *      scale_map [max_rows], red_map [max_rows*k] (sentinel R*k), ret_incl [W*S]
 * scale_map/red_map/ret_incl may be NULL together to compute only the GEMM plan.
 * status: optional int32[2] device words.  If the row count read from recv_incl
 *      is negative or exceeds max_rows (every buffer was sized from max_rows),
 *      nothing is sorted: excl and ret_incl are written as all zeros (no GEMM
 *      rows, nothing returned), status[0] = EPSB_PLAN_ROWS_EXCEEDED, status[1] =
 *      the offending count, and the maps are left untouched.  Zero it before the
 *      call; read it after synchronising. */
#define EPSB_PLAN_ROWS_EXCEEDED 51
int epsb_expert_plans(const int32_t* ridx, const int32_t* recv_incl, int k, int lo, int hi, int W, int S,
                      int max_tok_per_gpu, int64_t max_rows, int32_t* excl, int32_t* gemm_map, int32_t* inv_gemm,
                      int32_t* scale_map, int32_t* red_map, int32_t* ret_incl, int32_t* status, int max_cluster,
                      void* stream);

/* Same plans as epsb_expert_plans, for callers that are not allowed to allocate device memory.
 * This entry point has no counterpart in the reference.
 *
 * Who needs it: a host that was handed all of its buffers up front and must not call the allocator while it runs —
 * for example a serving loop whose memory is planned once per model (a cudaMalloc there would stall every stream of
 * the device), or a plug-in loaded by a runtime that owns the arena and gives the plug-in no allocation hook.  Such a
 * caller can provide the outputs but has nowhere to get the kernel's private scratch (the inverse GEMM map) from.
 *
 * Here that scratch is a fixed array inside the library's device image: 2^20 int32 entries (4 MiB), held by every GPU
 * that loads the library until the process exits.  Limits and rules:
 *   - max_rows * k must be <= 1048576, otherwise EPSB_ERR_WORKSPACE is returned and nothing is launched;
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine.  The FIRST call on a
 *     device is still special: it looks the array's device address up (cudaGetSymbolAddress, with that device
 *     current) and remembers it, and with CUDA's default lazy module loading that same call can be the moment the
 *     driver loads this library's device image onto the GPU, which is when the 4 MiB are actually reserved.  So
 *     the promise "nothing is allocated" holds from the second call on a device on: make one warm-up call per
 *     device during set-up, before any stream capture begins;
 *   - the remembered address belongs to the device's current primary context: after cudaDeviceReset (or any
 *     other teardown of that context) it is stale and this entry point must not be used in the process again;
 *   - a row count on the device that exceeds max_rows is refused like in epsb_expert_plans (status word), so the
 *     kernel never writes past the array;
 *   - every call on a device shares the one array: two calls whose kernels overlap on the GPU (different streams)
 *     race on it.  Nothing in it has to start at zero — the kernel writes every entry it later reads — and after
 *     the call it simply holds the last call's inverse map.
 * Arguments are those of epsb_expert_plans without inv_gemm. */
int epsb_expert_plans_noalloc(const int32_t* ridx, const int32_t* recv_incl, int k, int lo, int hi, int W, int S,
                              int max_tok_per_gpu, int64_t max_rows, int32_t* excl, int32_t* gemm_map,
                              int32_t* scale_map, int32_t* red_map, int32_t* ret_incl, int32_t* status,
                              int max_cluster, void* stream);

/* ----------------------------------------------------------------------------
 * fast_ep plans.  ref: src/fast_ep/all_to_all/fast_ep_kernels.cu:40-176
 * (expandPlan) and :352-610 (allGatherPlan + planKernel).
 * -------------------------------------------------------------------------- */
int epsb_fastep_expand_plan(const int32_t* idx, int T, int k, int E, int32_t* excl, int32_t* mapping, void* stream);
int epsb_fastep_plan(const int32_t* all_gathered, int my_rank, int W, int E, int32_t* remote_recv_plan,
                     int32_t* local_send_plan, int32_t* gemm_plan, int32_t* arr_src, int32_t* arr_rows,
                     int32_t* arr_dst, void* stream);

/* ----------------------------------------------------------------------------
 * Row movement.  row_bytes % 16 == 0 and all row bases 16-byte aligned, except
 * epsb_gather_rows which also takes rows of any multiple of 4 bytes (the [k]
 * index / weight rows).
 * -------------------------------------------------------------------------- */

/* dst[i,:] = src[(map[i] / map_div) % map_mod, :] for i in [begin, end) where
 * begin = bounds ? bounds[b0] : 0 and end = bounds ? bounds[b1] : n_rows
 * (bounds read on the device; max_rows bounds the grid).
 * ref: expandForComm (src/scheduler/comm_expander.cu:118-215; map_div 1,
 *      map_mod T) and expandForGemm (src/scheduler/gemm_expander.cu:81-163;
 *      map_div k, map_mod INT32_MAX, bounds = exclusive_sum). */
int epsb_gather_rows(const void* src, void* dst, const int32_t* map, int32_t map_div, int32_t map_mod,
                     const int32_t* bounds, int b0, int b1, int64_t n_rows, int64_t max_rows, int64_t row_bytes,
                     void* stream);

/* dst[map[i], :] = src[i / div, :] for i < n, skipping map[i] >= 1000000.
 * ref: fast_ep expand (fast_ep_kernels.cu:179-214). */
int epsb_scatter_rows(const void* src, void* dst, const int32_t* map, int32_t div, int64_t n, int64_t row_bytes,
                      void* stream);

/* Segment copy: for p < n_seg, rows [src_off[p], +rows[p]) -> [dst_off[p], ...).
 * ref: fast_ep arrange (fast_ep_kernels.cu:653-690). */
int epsb_arrange_rows(const void* src, void* dst, const int32_t* src_off, const int32_t* rows, const int32_t* dst_off,
                      int n_seg, int64_t max_rows, int64_t row_bytes, void* stream);

/* ----------------------------------------------------------------------------
 * Reductions.  H % 8 == 0.
 * -------------------------------------------------------------------------- */

/* Reference-arithmetic local reduce: send[q,:] = sum_j bf16(w[scale_map[q],j]) *
 * y[red_map[q,j],:] in bf16 multiply / bf16 accumulate, for q in the stage
 * window of every source rank.
 * ref: localReduce (src/scheduler/local_reducer.cu:103-211). stage -1 = all. */
int epsb_local_reduce_ref(const void* y, const float* w_recv, const int32_t* scale_map, const int32_t* red_map,
                          const int32_t* ret_incl, int k, int W, int S, int stage, int64_t max_rows, int64_t H,
                          void* send, void* stream);

/* Fast local reduce for the fused path: y rows are already weighted (fp32, in
 * the down-GEMM epilogue); send[q,:] = bf16(sum_j float(y[red_map[q,j],:])),
 * fp32 accumulation in slot order. */
int epsb_local_reduce(const void* y, const int32_t* red_map, const int32_t* ret_incl, int k, int W, int S, int stage,
                      int64_t max_rows, int64_t H, void* send, void* stream);

/* Reference-arithmetic global reduce + zero-expert term:
 * out[t,:] = (shared[t,:] +) sum_ep recv[glob_map[t,ep],:] in bf16 adds, then
 * out += bf16(float(x[t,:]) * zero_scale[t]) when zero_scale != NULL.
 * ref: globalReduce (src/scheduler/global_reducer.cu:126-208),
 *      zeroReduce (src/scheduler/zero_reducer.cu:34-50). */
int epsb_global_reduce_ref(const void* recv, const int32_t* glob_map, const void* shared, const void* x,
                           const float* zero_scale, int T, int W, int64_t H, void* out, void* stream);

/* Fused form: one fp32 accumulation, one bf16 rounding. */
int epsb_global_reduce(const void* recv, const int32_t* glob_map, const void* shared, const void* x,
                       const float* zero_scale, int T, int W, int64_t H, void* out, void* stream);

/* World of one (ep_world_size == 1): local reduce, the (empty) exchange and the global reduce in one pass.
 * out[t,:] = bf16(sum_j float(y[red_map[q,j],:]) (+shared[t,:]) (+x[t,:]*zero_scale[t])), q = glob_map[t],
 * y rows pre-weighted, fp32 accumulation in slot order, one rounding.
 * ref: the chain localReduce -> All2All -> globalReduce -> zeroReduce (src/scheduler/scheduler.cu:171-228)
 * when every peer is the rank itself. */
int epsb_reduce_ep1(const void* y, const int32_t* red_map, const int32_t* glob_map, const int32_t* ret_incl, int S,
                    const void* shared, const void* x, const float* zero_scale, int T, int k, int64_t H, void* out,
                    void* stream);

/* fast_ep combine: out[t,:] = bf16(sum_j w[t,j]*row(mapping[t*k+j]) (+shared)),
 * fp32 FMA accumulation; mapping >= 1000000 reads raw token mapping-1000000.
 * ref: fast_ep reduce (fast_ep_kernels.cu:231-335). */
int epsb_fastep_reduce(const void* rows, const void* raw, const void* shared, const float* w, const int32_t* mapping,
                       int T, int k, int64_t H, void* out, void* stream);

/* ----------------------------------------------------------------------------
 * SwiGLU (unfused, bf16 callers).  ref: silu_activate
 * (src/executor/activations.cu:9-40,173-205; src/executor/bindings/silu_ops.cu:14-43).
 * gate_up [rows, 2I] bf16 ([gate | up]) -> act [rows, I] bf16 over rows
 * [exclusive_sum[0], exclusive_sum[num_experts]) (or all `rows` if NULL).
 * -------------------------------------------------------------------------- */
int epsb_silu_run(const void* gate_up, void* act, const int32_t* exclusive_sum, int num_experts, int64_t rows,
                  int64_t inter_size, void* stream);

/* ----------------------------------------------------------------------------
 * FP8 block-scaled grouped GEMM (tcgen05 + TMEM, persistent ragged-M scheduler).
 * ref: GemmInterface::run (src/scheduler/gemm_executor_interface.cuh:3-29),
 *      AokGroupedGemm::run (src/executor/aok_grouped_gemm.cu:22-37),
 *      SM90_GROUPED_GEMM::Launch (src/gemm/aok_grouped_gemm/src/operations/
 *      hopper_grouped_gemm_kernel.h:322-400).  The A_scales / weight_scales
 *      slots of RunParams are the a_s / b_s arguments here.
 *
 * For local expert e, rows [excl[e], excl[e+1]) of A:
 *   C[m,n] = sum_kb a_s[m,kb] * b_s[e, n/128, kb] * sum_{k in kb} A[m,k]*B[e,n,k]
 * A   [max_rows, K] e4m3 row-major; a_s [max_rows, K/128] fp32 row-major
 * B   [EL, N, K] e4m3 (K contiguous); b_s [EL, N/128, K/128] fp32
 * excl [EL+1] int32 on the device (never read on the host)
 * K % 128 == 0, N % 128 == 0.
 *
 * status: optional int32[4] device words; word 0 is set nonzero if a bounded
 * device-side wait expired (the kernel then drains and exits instead of
 * hanging); word 1 holds the CTA that gave up.  Read it after synchronising.
 *
 * mode EPSB_GEMM_PLAIN : C [max_rows, N] bf16 = result.
 * mode EPSB_GEMM_GATEUP: N = 2I, B rows are [gate(I) | up(I)] (activations.cu:19-20);
 *      act = silu(gate)*up in fp32, requantised per row per 128 columns:
 *      C is e4m3 [max_rows, I], c_s [max_rows, I/128] fp32.  I % 128 == 0.
 * mode EPSB_GEMM_DOWN  : C [max_rows, N] bf16 = result * row_w[m] (fp32), the
 *      top-k gate weight of GEMM row m; row_w NULL = 1.
 * -------------------------------------------------------------------------- */
/* sm_count: SMs this launch of the persistent kernel may occupy (one CTA each);
 * 0 = all of them.  ref: the sm_count argument of aok_create
 * (src/executor/aok_grouped_gemm.cu:12,34, src/executor/bindings/aok_grouped_gemm_ops.cu).
 * A caller passes less than all to leave SMs to a kernel running on another stream. */
#define EPSB_GEMM_PLAIN 0
#define EPSB_GEMM_GATEUP 1
#define EPSB_GEMM_DOWN 2
int epsb_grouped_gemm_fp8(int mode, const void* A, const float* a_s, const void* B, const float* b_s,
                          const int32_t* excl, int num_experts, int64_t max_rows, int64_t N, int64_t K, void* C,
                          float* c_s, const float* row_w, int32_t* status, int sm_count, void* stream);

/* The same product with index-driven A loads: GEMM row m is row a_rows[m] of the a_src_rows x K matrix A_src (and of
 * a_s_src), fetched by the kernel's TMA producer four rows at a time (tile::gather4).  This replaces the separate
 * gather pass into an expert-contiguous A buffer (ref: expandForGemm, src/scheduler/gemm_expander.cu:81-163): the
 * rows are read where they arrived (or, in a world of one, where the quantiser wrote them).  a_rows [max_rows] int32
 * on the device (epsb_gemm_row_sources writes it); every other argument as in epsb_grouped_gemm_fp8. */
int epsb_grouped_gemm_fp8_gather(int mode, const void* A_src, const float* a_s_src, int64_t a_src_rows,
                                 const int32_t* a_rows, const void* B, const float* b_s, const int32_t* excl,
                                 int num_experts, int64_t max_rows, int64_t N, int64_t K, void* C, float* c_s,
                                 const float* row_w, int32_t* status, int sm_count, void* stream);

/* Source row and gate weight of every GEMM row d < excl[num_experts], from the GEMM plan (gemm_map[d] = received row *
 * k + slot): a_rows[d] = the received row, or with send_map (a world of one: the receive order is the send order) the
 * token behind it, send_map[row] % T; row_w[d] = w_src[a_rows[d] * k + slot] (NULL to skip).  w_src is the received
 * gate weights [R, k], or in a world of one the caller's expert_scales [T, k]. */
int epsb_gemm_row_sources(const int32_t* gemm_map, const int32_t* excl, int num_experts, int k, const int32_t* send_map,
                          int T, const float* w_src, int64_t max_rows, int32_t* a_rows, float* row_w, void* stream);

/* bf16 x bf16 -> bf16 grouped GEMM (tcgen05 kind::f16, accumulators resident in TMEM over the whole K extent):
 * for local expert e, C[m,:] = A[m,:] * B[e]^T over rows [excl[e], excl[e+1]), fp32 accumulation, one rounding.
 * ref: AokGroupedGemm::run (src/executor/aok_grouped_gemm.cu:22-37), the op executor.aok_run
 *      (src/executor/bindings/aok_grouped_gemm_ops.cu:39-84), SM90_GROUPED_GEMM::Launch
 *      (src/gemm/aok_grouped_gemm/src/operations/hopper_grouped_gemm_kernel.h:322-400; alpha 1, beta 0).
 * A [max_rows, K] bf16 row-major, B [EL, N, K] bf16 (K contiguous), C [max_rows, N] bf16.  K % 64 == 0, N % 128 == 0.
 * excl, status, sm_count as in epsb_grouped_gemm_fp8.  No workspace (aok_get_workspace_size is 0).
 * rows_hint: the number of rows the caller expects (the reference's num_tokens_hint; 0 = unknown, max_rows is used).
 * It only picks the tile form: with at least 512 expected rows per expert and N % 256 == 0, pairs of CTAs compute
 * 256 x 256 tiles (tcgen05.mma.cta_group::2, each CTA stages half of the weight rows), else single CTAs 128 x 256. */
int epsb_grouped_gemm_bf16(const void* A, const void* B, const int32_t* excl, int num_experts, int64_t max_rows,
                           int64_t rows_hint, int64_t N, int64_t K, void* C, int32_t* status, int sm_count,
                           void* stream);

/* Gathers the per-GEMM-row gate weight: row_w[d] = w_recv[gemm_map[d]] for
 * d < excl[EL] (w_recv is [R,k] flat, gemm_map holds row*k+slot). */
int epsb_gather_row_weights(const float* w_recv, const int32_t* gemm_map, const int32_t* excl, int num_experts,
                            int64_t max_rows, float* row_w, void* stream);

/* ----------------------------------------------------------------------------
 * Expert-parallel exchange over peer memory (one NVSwitch box, W <= 8 ranks).
 * ref: CommBuffs arenas (src/communication/msccl_comm.cu:191-255), the plan
 *      all-gather with flags and getRecvPlan (src/communication/alltoall_runner.cu:39-128),
 *      the SM-copy all-to-all All2All<T> (alltoall_runner.cu:131-256, smChan_put in
 *      src/communication/msccl_comm.cuh:166-183); fused with expandForComm
 *      (src/scheduler/comm_expander.cu:118-215) on the way out and with localReduce
 *      (src/scheduler/local_reducer.cu:103-211) on the way back.
 *
 * Every rank owns one symmetric REGION that all ranks of the box map (CUDA IPC):
 * plan tables, flag words and the receive arenas.  After set-up nothing goes
 * through the host: plans are stored into the peers' tables and announced with a
 * flag, rows are stored by SM threads straight into the destination's arena at
 * the offset the exchanged plans give, and each exchange ends with a flag at
 * every peer.  Only peer STORES are used (no loads from peer memory, no TMA, no
 * multicast).  Flags carry the call's epoch, which only grows; tables and
 * dispatch arenas are double-buffered by epoch parity.
 * Every spin is bounded: after timeout_ns (<= 0: EPSB_EXCHANGE_DEFAULT_TIMEOUT_NS)
 * the kernel writes a code into status[0] (and the peer it waited for into
 * status[1]) and returns; after a plan time-out the exchange of that call is
 * empty (all counts 0), so the later kernels of the call are no-ops.
 * -------------------------------------------------------------------------- */
#define EPSB_MAX_PEERS 8
#define EPSB_IPC_HANDLE_BYTES 64
#define EPSB_EXCHANGE_DEFAULT_TIMEOUT_NS 2000000000ll
#define EPSB_EXCHANGE_TIMEOUT_PLANS 61  /* status code: a peer's plans did not arrive */
#define EPSB_EXCHANGE_ROWS_EXCEEDED 62  /* status code: the peers announce more rows than the arena holds */
#define EPSB_EXCHANGE_TIMEOUT_DATA 70   /* status code base: + flag slot of the exchange that did not complete */

/* Symmetric memory.  epsb_symm_alloc: cudaMalloc + zero fill + IPC handle (64 bytes, to be sent to the peers by
 * whatever channel the host has); epsb_symm_open maps a peer's handle into this process.  These four functions
 * allocate / free device memory and synchronise; they belong to set-up and tear-down. */
int epsb_symm_alloc(int64_t bytes, void** ptr, uint8_t* handle64);
int epsb_symm_open(const uint8_t* handle64, void** ptr);
int epsb_symm_close(void* ptr);
int epsb_symm_free(void* ptr);

typedef struct epsb_exchange epsb_exchange_t;

/* Size of one rank's region for (W ranks, max_tok tokens per rank, up to S_max stages, top-k, hidden size H with
 * elements of hidden_elem_bytes (1 = e4m3 codes, 2 = bf16), scales_dim fp32 scales per row (0 = none)): arenas of
 * max_tok * W rows each, as the reference sizes them (msccl_comm.cu:191-199). */
int epsb_exchange_region_bytes(int W, int max_tok, int S_max, int k, int64_t H, int hidden_elem_bytes, int scales_dim,
                               int64_t* bytes);
/* peer_regions: host array of W device pointers, entry r = rank r's region as mapped into this process (entry
 * `rank` = this rank's own allocation).  Allocates a few hundred bytes of device scratch (set-up). */
int epsb_exchange_create(int rank, int W, int max_tok, int S_max, int k, int64_t H, int hidden_elem_bytes,
                         int scales_dim, void* const* peer_regions, epsb_exchange_t** out);
int epsb_exchange_destroy(epsb_exchange_t* x);
/* Starts the next call: advances the epoch (host side, no launch).  Every rank must go through the same sequence
 * of begin / publish / recv_plans / put / wait / local_reduce_put calls. */
int epsb_exchange_begin(epsb_exchange_t* x, int* epoch);

#define EPSB_ARENA_IDX 0       /* int32 [rows, k]   received expert ids */
#define EPSB_ARENA_WEIGHTS 1   /* fp32  [rows, k]   received gate weights */
#define EPSB_ARENA_HIDDEN 2    /* [rows, H]         received hidden rows */
#define EPSB_ARENA_SCALES 3    /* fp32  [rows, scales_dim] */
#define EPSB_ARENA_OUT 4       /* bf16  [rows, H]   returned partial rows (collect arena) */
#define EPSB_ARENA_RECV_PLAN 5 /* int32 [W * S_max] the receive plan epsb_exchange_recv_plans derived */
/* Device address of one of this rank's arenas; parity = epoch & 1 for the double-buffered ones. */
int epsb_exchange_arena(epsb_exchange_t* x, int which, int parity, void** ptr);

/* send_incl / coll_incl [W*S]: the plans epsb_source_plans wrote.  One CTA; stores + one flag per peer. */
int epsb_exchange_publish_plans(epsb_exchange_t* x, const int32_t* send_incl, const int32_t* coll_incl, int S,
                                void* stream);
/* Waits for every peer's plans, then derives the receive plan (also copied to recv_incl [W*S] if not NULL;
 * ref getRecvPlan, alltoall_runner.cu:60-101) and this rank's landing offsets at every peer for both directions. */
int epsb_exchange_recv_plans(epsb_exchange_t* x, int S, int32_t* recv_incl, int32_t* status, int64_t timeout_ns,
                             void* stream);

/* Flag slots of the data exchanges (slot 0 is the plans'). */
#define EPSB_FLAG_META 1
#define EPSB_FLAG_DISPATCH(stage) (2 + (stage))
#define EPSB_FLAG_COMBINE(S_max, stage) (2 + (S_max) + (stage))
#define EPSB_PUT_META 1    /* expert ids + gate weights */
#define EPSB_PUT_SCALES 2
#define EPSB_PUT_HIDDEN 4
/* Permute-on-send: rows of the send order whose stage is `stage` (all stages if < 0) are read through send_map
 * (row i is token send_map[i] % T) and stored into their destination's arenas; `mask` selects the arrays.  The
 * last CTA releases flag `flag_slot` at every peer.  idx [T,k], weights [T,k], hidden [T,H], scales [T,scales_dim]. */
int epsb_exchange_put(epsb_exchange_t* x, int flag_slot, int stage, int mask, const int32_t* idx, const float* weights,
                      const void* hidden, const float* scales, const int32_t* send_map, const int32_t* send_incl, int T,
                      int S, void* stream);
/* Consumer side of an exchange: bounded wait for flag `flag_slot` of every peer (one warp). */
int epsb_exchange_wait(epsb_exchange_t* x, int flag_slot, int32_t* status, int64_t timeout_ns, void* stream);
/* Return trip: epsb_local_reduce (pre-weighted rows, fp32 accumulation) whose output row lands directly in the
 * source rank's collect arena; then flag `flag_slot` at every peer. */
int epsb_exchange_local_reduce_put(epsb_exchange_t* x, int flag_slot, const void* y, const int32_t* red_map,
                                   const int32_t* ret_incl, int S, int stage, int64_t max_rows, void* stream);

/* ----------------------------------------------------------------------------
 * fast_oep: lookups in an embedding table sharded over the ranks (rank r owns ids [r * size_per_rank, (r+1) *
 * size_per_rank)).  ids travel to their owners, table rows travel back.
 * ref: FastOEP<T>::dispatch / combine (src/fast_oep/all_to_all/fast_oep.cu:52-151), arrangeAndPlanKernel,
 *      lookupKernel, scatterKernel (src/fast_oep/all_to_all/fast_oep_kernels.cu:15-58,186-245).
 * Built on the exchange above, created with k = 1, H = embed_dim, hidden_elem_bytes = 0 (no hidden arenas),
 * scales_dim = 0, S_max = 1 and max_tok * W >= the ids all ranks hold together:
 *   dispatch  epsb_oep_arrange_plan; epsb_exchange_begin; publish_plans(send_incl, send_incl, 1); recv_plans;
 *             epsb_exchange_put_ids(EPSB_FLAG_META); epsb_exchange_wait(EPSB_FLAG_META)
 *   combine   epsb_exchange_lookup_put(EPSB_FLAG_COMBINE(1, 0)); epsb_exchange_wait(same); epsb_oep_scatter from
 *             the EPSB_ARENA_OUT rows.
 * epsb_oep_arrange_plan: stable counting sort of the ids by owner (the reference hands out positions with atomics,
 * so its order inside an owner's block is arbitrary; the looked-up result does not depend on it).  send_incl [W]
 * inclusive counts per owner, mapping [n]: id i -> its position in the arranged order or -1 (negative ids, and ids
 * beyond the table, are skipped: their output rows are left untouched), send_map [n]: the inverse.
 * -------------------------------------------------------------------------- */
int epsb_oep_arrange_plan(const int32_t* ids, int64_t n, int64_t size_per_rank, int W, int32_t* send_incl,
                          int32_t* mapping, int32_t* send_map, void* stream);
int epsb_exchange_put_ids(epsb_exchange_t* x, int flag_slot, const int32_t* ids, const int32_t* send_map,
                          const int32_t* send_incl, int64_t n, void* stream);
/* table: this rank's shard [size_per_rank, embed_dim] bf16; row id % size_per_rank answers a received id. */
int epsb_exchange_lookup_put(epsb_exchange_t* x, int flag_slot, const void* table, int64_t size_per_rank,
                             int64_t max_rows, void* stream);
/* out[dst(i), :] = rows[mapping[i], :] for mapping[i] >= 0, dst(i) = i or, with do_permute, the n-gram-major position
 * i / n_grams + (i % n_grams) * (n / n_grams). */
int epsb_oep_scatter(const void* rows, const int32_t* mapping, int64_t n, int64_t row_bytes, int64_t n_grams,
                     int do_permute, void* out, void* stream);

/* ----------------------------------------------------------------------------
 * TP <-> DP conversion of [tokens, hidden] bf16 rows inside a tensor-parallel
 * group of the box (the step either side of the MoE block in a model whose
 * attention is tensor-parallel).
 * ref: TPDPConvertor (src/communication/tp_dp_convertor.cu:54-129),
 *      AllGatherRunner (src/communication/allgather_runner.cu:13-83),
 *      ReduceScatterRunner (src/communication/reducescatter_runner.cu:61-122).
 * Every rank of the group owns one symmetric region (epsb_symm_alloc) of
 * epsb_tpdp_region_bytes: buffer_rows x buffer_hidden bf16 (the reference sizes
 * it attn_tp_size * tp_max_num_tokens rows) followed by flag words.  A call works
 * on tp_num_tokens rows of `hidden` (<= buffer_hidden) columns; rank r owns rows
 * [offset_r, offset_r + n_r), n_r = tp_num_tokens / tp_size (+1 for the first
 * tp_num_tokens % tp_size ranks), the reference's split (tp_dp_convertor.cu:54-62).
 * regions: host array of tp_size device pointers, entry r = rank r's region as
 * mapped here.  One collective is four launches on every rank, with `epoch` a
 * number that grows with every collective of the group:
 *   all-gather      signal(slot 0) wait(slot 0) all_gather_put(slot 1) wait(slot 1)
 *   reduce-scatter  signal(slot 2) wait(slot 2) reduce_scatter_sum(slot 3) wait(slot 3)
 * "ready" (even slot): my buffer holds my input and I no longer read anybody's
 * previous result; the data kernel releases the odd slot at every peer when its
 * last CTA is done.  all_gather_put uses peer stores, reduce_scatter_sum peer
 * loads (fp32 sum in rank order, so every rank would get the same bits).
 * A wait that runs out of time writes EPSB_TPDP_TIMEOUT + slot into status[0].
 * -------------------------------------------------------------------------- */
#define EPSB_TPDP_TIMEOUT 80
int epsb_tpdp_region_bytes(int64_t buffer_rows, int64_t buffer_hidden, int64_t* bytes);
int epsb_tpdp_signal(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows, int64_t buffer_hidden, int slot,
                     int epoch, void* stream);
int epsb_tpdp_wait(const void* my_region, int tp_size, int64_t buffer_rows, int64_t buffer_hidden, int slot, int epoch,
                   int32_t* status, int64_t timeout_ns, void* stream);
int epsb_tpdp_all_gather_put(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows, int64_t tp_num_tokens,
                             int64_t hidden, int64_t buffer_hidden, int slot, int epoch, void* stream);
int epsb_tpdp_reduce_scatter_sum(void* const* regions, int tp_rank, int tp_size, int64_t buffer_rows,
                                 int64_t tp_num_tokens, int64_t hidden, int64_t buffer_hidden, int slot, int epoch,
                                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EPS_B200_H_ */
