/*
 * C-ABI of libaiter_b200.so: the FP8 block-scaled fused-MoE path for NVIDIA B200 (sm_100a).
 *
 * Calling convention (the one ROCm/aiter's ctypes FFI binds, aiter/jit/core.py:1306-1620):
 *   - every entry point returns int: 0 = success, -1 = failure; the message of the last
 *     failure on the calling thread is read with aiter_get_last_error()
 *     (csrc/include/aiter_ctypes_error.h:55-155);
 *   - tensors travel as pointers to the 160-byte POD aiter_tensor_t
 *     (csrc/include/aiter_tensor.h:8-18); an absent optional tensor is NULL;
 *   - the caller owns every buffer (inputs, outputs and workspaces); the library never
 *     allocates, frees or retains device memory, and never synchronises the host;
 *   - the CUDA stream is the last argument (NULL = the legacy default stream); work is
 *     enqueued on the device that holds the first tensor argument.
 *
 * All tensors must be contiguous.  Paths are relative to the ROCm/aiter tree.
 */
#ifndef AITER_B200_H
#define AITER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* csrc/include/aiter_enum.h:36-52 */
typedef enum {
    AITER_DTYPE_fp8 = 0,
    AITER_DTYPE_fp8_e8m0,
    AITER_DTYPE_fp16,
    AITER_DTYPE_bf16,
    AITER_DTYPE_fp32,
    AITER_DTYPE_i4x2,
    AITER_DTYPE_fp4x2,
    AITER_DTYPE_u32,
    AITER_DTYPE_i32,
    AITER_DTYPE_i16,
    AITER_DTYPE_i8,
    AITER_DTYPE_u8,
    AITER_DTYPE_i64,
    AITER_DTYPE_u64
} AiterDtype;

/* csrc/include/aiter_tensor.h:8-18 */
typedef struct aiter_tensor_t {
    void*   ptr;        /* device pointer                     */
    size_t  numel_;     /* number of elements                 */
    int     ndim;       /* number of dimensions (<= 8)        */
    int64_t shape[8];
    int64_t strides[8]; /* in elements                        */
    int     dtype_;     /* AiterDtype                         */
    int     device_id;  /* CUDA device index, -1 = host       */
} aiter_tensor_t;

/* csrc/include/aiter_ctypes_error.h:61-71 */
int         aiter_ctypes_abi_version(void); /* == 4 */
const char* aiter_get_last_error(void);     /* NULL when no error is pending */
void        aiter_clear_last_error(void);

/* Bytes of scratch b200_moe_sorting_fwd needs for this problem (0 when the single-CTA
 * path is taken).  Replaces moe_sorting_opus_get_workspace_size
 * (aiter/ops/moe_sorting_opus.py:12-18, csrc/include/moe_sorting_opus.h:1385-1427). */
int64_t b200_moe_sorting_get_workspace_size(int tokens, int num_experts, int topk, int dispatch_policy);

/* Stable counting sort of (token, slot) routes by expert, padded per expert to unit_size.
 * Replaces moe_sorting_opus_fwd (csrc/py_itfs_cu/moe_sorting_opus_kernels.cu:14-84,
 * argument order of aiter/ops/moe_sorting_opus.py:21-38).
 *   topk_ids [M,topk] i32, topk_weights [M,topk] fp32
 *   sorted_token_ids [P] i32 = slot<<24|token, pads = topk<<24|M   (P = M*topk + E*unit - topk)
 *   sorted_weights [P] fp32 (0 in pads), sorted_expert_ids [ceil(P/unit)] i32 (local ids, -1 past the end)
 *   num_valid_ids [2] i32 = {padded total, tokens sorted}
 *   moe_buf: optional [M, model_dim] buffer that is zero-filled (any dtype)
 *   local_expert_mask: optional [E] i32, 0 drops the expert and renumbers the others
 *   num_local_tokens: optional [1] i32 read on the device (rows >= it are ignored)
 *   workspace: >= b200_moe_sorting_get_workspace_size bytes when that is > 0
 *   local_topk_ids: optional [M,topk] i32 output, local expert id per route or -1
 *   m_indices, reverse_sorted: outputs of the reference's grouped-GEMM layout; not produced here, must be NULL */
int b200_moe_sorting_fwd(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                         aiter_tensor_t* sorted_token_ids, aiter_tensor_t* sorted_weights,
                         aiter_tensor_t* sorted_expert_ids, aiter_tensor_t* num_valid_ids,
                         aiter_tensor_t* moe_buf, int num_experts, int unit_size,
                         const aiter_tensor_t* local_expert_mask,
                         const aiter_tensor_t* num_local_tokens, aiter_tensor_t* workspace,
                         int dispatch_policy, aiter_tensor_t* local_topk_ids, aiter_tensor_t* m_indices,
                         aiter_tensor_t* reverse_sorted, void* stream);

/* No counterpart in the reference.  The same sort for callers that cannot allocate or pass a
 * workspace: a host runtime bound over an FFI that owns no device allocator, a serving loop whose
 * pool is frozen after start-up, or code that must avoid the device-wide synchronisation a
 * cudaMalloc/cudaFree implies.  The scratch lives in a fixed array inside the library
 * (266240 bytes, held by every GPU that loads it); problems that
 * need more (tokens*topk > 262144 routes) are rejected with an error.  Arguments as for
 * b200_moe_sorting_fwd without workspace and dispatch_policy.  The first call on a device resolves
 * the array's device address and should precede any stream capture.  Calls on the same device share
 * the array: do not let two of them overlap on the GPU. */
int b200_moe_sorting_fwd_noalloc(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                                 aiter_tensor_t* sorted_token_ids, aiter_tensor_t* sorted_weights,
                                 aiter_tensor_t* sorted_expert_ids, aiter_tensor_t* num_valid_ids,
                                 aiter_tensor_t* moe_buf, int num_experts, int unit_size,
                                 const aiter_tensor_t* local_expert_mask,
                                 const aiter_tensor_t* num_local_tokens, aiter_tensor_t* local_topk_ids,
                                 void* stream);

/* Dynamic per-row, per-128-column FP8 e4m3 quantisation: scale = amax/448 (1 when amax is 0),
 * codes = RNE(x / scale).  Replaces dynamic_per_token_scaled_quant with group_size=128
 * (aiter/ops/quant.py:439-483, csrc/kernels/quant_kernels.cu:27-167,720-830) with the
 * rounding sequence of the torch oracle (aiter/ops/quant.py:64-94).
 *   input [R,C] bf16|fp16 (C % 128 == 0) -> out [R,C] fp8, scales [R,C/128] fp32
 *   num_rows: optional [1] i32 on the device; only the first *num_rows * num_rows_factor rows are quantised
 *   transpose_scale != 0: the scale of (row, column group) is written at [column group * rows + row] of the same
 *   buffer (rows = the dynamic row count when num_rows is given), the layout the reference's 1-stage kernels read
 *   (shuffle_scale, csrc/kernels/quant_kernels.cu:143-146; aiter/fused_moe.py:1138-1147) */
int b200_moe_quant_1x128(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                         const aiter_tensor_t* num_rows, int num_rows_factor, int transpose_scale, void* stream);

/* Dynamic per-row FP8 e4m3 quantisation over the whole row (QuantType.per_Token): scale = amax/448
 * (1 when amax is 0), codes = RNE(x / scale). Replaces dynamic_per_token_scaled_quant
 * (aiter/ops/quant.py:406-436, csrc/kernels/quant_kernels.cu) with the rounding sequence of pertoken_quant
 * (aiter/ops/quant.py:64-94).
 *   input [R,C] bf16|fp16 -> out [R,C] fp8, scales [R] fp32; num_rows: optional [1] i32 on the device, rows >=
 *   *num_rows * num_rows_factor are skipped (the padded tail of a sorted buffer) */
int b200_moe_quant_per_token(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                             const aiter_tensor_t* num_rows, int num_rows_factor, void* stream);

/* Dynamic per-tensor FP8 e4m3 quantisation (QuantType.per_Tensor): scale = max|x| / 448, codes = RNE(x / scale).
 * Replaces dynamic_per_tensor_quant behind per_tensor_quant_hip (aiter/ops/quant.py:628-645) with the rounding
 * sequence of per_tensor_quant (aiter/ops/quant.py:318-328; like it, no guard for an all-zero tensor).
 *   input [R,C] bf16|fp16 -> out [R,C] fp8, scale [1] fp32; amax: [1] fp32 scratch word, cleared by the call;
 *   row_scales: optional [R] fp32, receives the scale once per row (the per_Token GEMM kernels take one scale per
 *   row); row_limit: optional [1] i32 on the device, rows >= it take no part (padded tail of a sorted buffer) */
int b200_moe_quant_per_tensor(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scale,
                              aiter_tensor_t* amax, aiter_tensor_t* row_scales, const aiter_tensor_t* row_limit,
                              void* stream);

/* Stage 1: grouped gate/up GEMM over the sorted blocks + SiLU(gate)*up + bf16 rounding +
 * 1x128 FP8 requantisation.  Replaces ck_moe_stage1 followed by the a2 quant
 * (csrc/ck_gemm_moe_2stages_codegen/gemm_moe_ck2stages.cu:68-137, aiter/fused_moe.py:3220-3336).
 * The sort must have used unit_size == 128.
 *   a1 [M,H] fp8 + a1_scale [M,H/128] fp32; w1 [E,2I,H] fp8 (gate rows then up rows) +
 *   w1_scale [E,2I/128,H/128] fp32
 *   a2 [P,I] fp8 and a2_scale [P,I/128] fp32, rows in SORTED order (row p belongs to
 *   sorted_token_ids[p]; rows of pads are zero)
 *   status [1] i32 device word: set non-zero if a bounded device-side wait ran out
 *   quant_type: QuantType (csrc/include/aiter_enum.h:16-26). 4/5 (per_1x128/per_128x128) as described; 2
 *   (per_Token): a1_scale [M], w1_scale [E,2I] (one per output channel), a2 is bf16 [P,I] (SiLU*up, rounded,
 *   sorted order) and a2_scale is NULL - the caller requantises rows with b200_moe_quant_per_token.
 *   sorted_weights: NULL, or the route weights to multiply the GEMM result with before the activation
 *   (doweight_stage1, aiter/fused_moe.py:3651-3652); activation: ActivationType, 0 = Silu, 1 = Gelu. */
int b200_moe_stage1(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale,
                    const aiter_tensor_t* w1, const aiter_tensor_t* w1_scale,
                    const aiter_tensor_t* sorted_token_ids, const aiter_tensor_t* sorted_expert_ids,
                    const aiter_tensor_t* num_valid_ids, aiter_tensor_t* a2, aiter_tensor_t* a2_scale,
                    aiter_tensor_t* status, int quant_type, const aiter_tensor_t* sorted_weights, int activation,
                    void* stream);

/* Stage 2: grouped down GEMM over the sorted blocks, times the route weight, accumulated
 * per token in fp32.  Replaces ck_moe_stage2
 * (csrc/ck_gemm_moe_2stages_codegen/gemm_moe_ck2stages.cu:139-199).
 *   a2/a2_scale as written by stage 1; w2 [E,H,I] fp8 + w2_scale [E,H/128,I/128] fp32
 *   acc [M, col_end-col_begin] fp32 (the range's own block) or [M, model_dim] (the whole buffer, of which columns
 *   [col_begin, col_end) are filled), zero on entry; receives sum over routes of weight * (a2 . w2)
 *   for the output columns [col_begin, col_end) (multiples of 256; col_end <= 0 means model_dim). Launching
 *   the columns in several ranges lets a caller hand finished ranges to a collective while the next is computed;
 *   sm_margin SMs are then left idle by this launch so that the collective's kernels can run beside it.
 *   quant_type 2 (per_Token): a2_scale [P], w2_scale [E,H]. doweight 0 leaves the route weight out
 *   (it was applied in stage 1). */
int b200_moe_stage2(const aiter_tensor_t* a2, const aiter_tensor_t* a2_scale,
                    const aiter_tensor_t* w2, const aiter_tensor_t* w2_scale,
                    const aiter_tensor_t* sorted_token_ids, const aiter_tensor_t* sorted_weights,
                    const aiter_tensor_t* sorted_expert_ids, const aiter_tensor_t* num_valid_ids,
                    aiter_tensor_t* acc, aiter_tensor_t* status, int col_begin, int col_end, int sm_margin,
                    int quant_type, int doweight, void* stream);

/* out[M,H] (bf16 or fp16) = round-to-nearest-even(acc[M,H] fp32): the single final rounding of
 * the reference's `out.sum(1).to(dtype)` (aiter/fused_moe.py:3811). */
int b200_moe_finalize(aiter_tensor_t* out, const aiter_tensor_t* acc, void* stream);

/* Expert-parallel combine over NVLink peer memory, in place of a dense fp32 reduce-scatter of the [M,H]
 * partial sums. The reference's counterparts are MoRI's combine and the stage-2 scatter epilogue into a
 * peer-memory arena (`Stage2ScatterContext`, aiter/fused_moe.py:536-575; oracle
 * op_tests/multigpu_tests/test_dispatch_combine.py:18-72).
 *   b200_ep_dispatch: the quantised row of every local token (a1 [m_local,H] fp8, a1_scale [m_local,H/128] fp32) is
 *     stored at the token's global row (rank*m_local + row) of the a1 / a1_scale buffers ([M,H], [M,H/128]) of every
 *     rank that holds one of the experts in topk_ids[row,:] (i32 [m_local,topk], GLOBAL ids); peer_a1 and
 *     peer_a1_scale are i64 [world] device arrays with those buffers' addresses as mapped in this process (the
 *     rank's own buffers included). Takes the place of the all-gather of the tokens; rows a rank has no route
 *     for are not sent (and never read by its stage 1).
 *   b200_ep_push_partials: rank `rank` copies acc[t,:] (fp32 [M,H], M = world * m_local) of every token t owned
 *     by another rank o for which topk_ids[t,:] (i32 [M,topk], GLOBAL expert ids) names one of its experts
 *     (id / experts_per_rank == rank) into recv_o[rank, t - o*m_local, :]; peer_recv is an i64 [world] device
 *     array with the address of every rank's recv buffer (fp32 [world, m_local, H]) as mapped in this process.
 *   The caller then runs any collective as a barrier, and
 *   b200_ep_combine: out[tl,:] (bf16/fp16 [m_local,H]) = round(sum over ranks r, ascending, that have a route of
 *     token t = rank*m_local + tl, of (r == rank ? acc[t,:] : recv[r,tl,:])).
 *   b200_ep_ipc_export / _open / _close: CUDA IPC for the receive buffers. export writes the 64-byte handle of the
 *     allocation that holds `tensor` and the tensor's byte offset in it; open maps such a handle from another
 *     process for kernels of `device` (the mapping belongs to the device that is current while it is opened, so
 *     every rank opens its peers' handles under its own device) and returns the base address; close unmaps it.
 * expert_rank: optional [global experts] i32, the rank that owns each expert, for placements that are not contiguous
 *     slices (NULL: expert e lives on rank e / experts_per_rank).
 * No device-side waiting between ranks; rows that were not pushed are never read. */
int b200_ep_dispatch(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale, const aiter_tensor_t* topk_ids,
                     const aiter_tensor_t* peer_a1, const aiter_tensor_t* peer_a1_scale, int rank, int world,
                     int experts_per_rank, const aiter_tensor_t* expert_rank, void* stream);
/* The same dispatch fused with the 1x128 quantisation that precedes it (b200_moe_quant_1x128's arithmetic): input
 * [M/G, model_dim] bf16 or fp16; the codes and scales go straight into the peers' buffers. */
int b200_ep_quant_dispatch(const aiter_tensor_t* input, const aiter_tensor_t* topk_ids, const aiter_tensor_t* peer_a1,
                           const aiter_tensor_t* peer_a1_scale, int rank, int world, int experts_per_rank,
                           const aiter_tensor_t* expert_rank, void* stream);
/* col_begin/col_end: push only these columns of every row (0, 0 = all), so that a finished column range of stage 2
 * can travel while the next range is computed; sm_limit > 0 bounds the launch to that many SMs' worth of CTAs. */
int b200_ep_push_partials(const aiter_tensor_t* acc, const aiter_tensor_t* topk_ids, const aiter_tensor_t* peer_recv,
                          int rank, int world, int experts_per_rank, const aiter_tensor_t* expert_rank, int col_begin,
                          int col_end, int sm_limit, void* stream);
int b200_ep_combine(aiter_tensor_t* out, const aiter_tensor_t* acc, const aiter_tensor_t* recv,
                    const aiter_tensor_t* topk_ids, int rank, int world, int experts_per_rank,
                    const aiter_tensor_t* expert_rank, void* stream);
int b200_ep_ipc_export(const aiter_tensor_t* tensor, void* handle_out, int64_t* offset_out);
int b200_ep_ipc_open(const void* handle, int device, int64_t* ptr_out);
int b200_ep_ipc_close(int64_t ptr, int device);

/* No counterpart in the reference (its kernels wait without a limit). Self-test hook of the bounded device-side
 * waits of the GEMM kernels: for every later stage-1/stage-2 launch of this process, wait_limit_cycles is the number
 * of SM clocks after which a wait gives up (<= 0 restores the built-in limit of about 2 s) and a non-zero
 * stall_weight_producer makes the weight-loading role issue nothing. With it stalled nothing is in flight, the waits run
 * out, every CTA winds down and frees its tensor memory, and the caller's status word is set to 1. Tests only. */
int b200_moe_debug_config(int64_t wait_limit_cycles, int stall_weight_producer);

/* DeepSeek-V3 style router: sigmoid scores, correction bias for the choice only, groups ranked by the sum
 * of their two best biased scores, top `topk_group` groups kept, top-k experts among them; weights are the
 * un-biased scores, renormalised when asked, times routed_scaling_factor. Replaces biased_grouped_topk
 * (aiter/ops/topk.py:89-99,176-215, csrc/kernels/topk_softmax_kernels_group.cu:1219-1266) with the arithmetic
 * of biased_grouped_topk_torch (aiter/ops/topk.py:217-259).
 *   gating_output [M,E] fp32|bf16, correction_bias [E] fp32|bf16 -> topk_weights [M,topk] fp32, topk_ids [M,topk] i32
 *   E <= 1024, topk <= 32, num_expert_group <= 32 and a divisor of E */
int b200_biased_grouped_topk(const aiter_tensor_t* gating_output, const aiter_tensor_t* correction_bias,
                             aiter_tensor_t* topk_weights, aiter_tensor_t* topk_ids, int num_expert_group,
                             int topk_group, int need_renorm, float routed_scaling_factor, void* stream);

/* fp32 softmax over the experts, top-k, optional renormalisation. Replaces topk_softmax
 * (aiter/ops/moe_op.py:29-66, csrc/kernels/topk_softmax_kernels.cu:769) as used by fused_topk
 * (aiter/fused_moe.py:4058-4129). token_expert_indices is optional ([M,topk] i32 = k*M + token). */
int b200_topk_softmax(aiter_tensor_t* topk_weights, aiter_tensor_t* topk_indices,
                      aiter_tensor_t* token_expert_indices, const aiter_tensor_t* gating_output,
                      int need_renorm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AITER_B200_H */
