// C-ABI entry points of libaiter_b200.so (declared in include/aiter_b200.h) and the error bridge.
// Conventions of the reference's ctypes FFI: int status, thread-local last-error string, stream as
// the last argument (csrc/include/aiter_ctypes_error.h:55-155, aiter/jit/core.py:1306-1620).

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

std::string& last_error() {
    static thread_local std::string msg;
    return msg;
}

int64_t sorting_workspace_bytes(int tokens, int num_experts, int topk);
void launch_moe_sorting(const aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*,
                        aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, int, int, const aiter_tensor_t*,
                        const aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, cudaStream_t);
void launch_moe_sorting_noalloc(const aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*,
                                aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, int, int, const aiter_tensor_t*,
                                const aiter_tensor_t*, aiter_tensor_t*, cudaStream_t);
void launch_quant_1x128(aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, const aiter_tensor_t*, int, int, cudaStream_t);
void launch_quant_per_token(aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, const aiter_tensor_t*, int, cudaStream_t);
void launch_quant_per_tensor(aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*,
                             const aiter_tensor_t*, cudaStream_t);
void launch_moe_stage1(const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*,
                       const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*,
                       aiter_tensor_t*, aiter_tensor_t*, int, const aiter_tensor_t*, int, cudaStream_t);
void launch_moe_stage2(const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*,
                       const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*,
                       aiter_tensor_t*, aiter_tensor_t*, int, int, int, int, int, cudaStream_t);

void set_gemm_debug(long long, int);

void launch_biased_grouped_topk(const aiter_tensor_t*, const aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, int, int,
                                int, float, cudaStream_t);
void launch_topk_softmax(aiter_tensor_t*, aiter_tensor_t*, aiter_tensor_t*, const aiter_tensor_t*, int, cudaStream_t);
void launch_ep_push(const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, int, int, int, const aiter_tensor_t*,
                    int, int, int, cudaStream_t);
void launch_ep_combine(aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, int, int, int,
                       const aiter_tensor_t*, cudaStream_t);
void launch_ep_quant_dispatch(const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, int,
                              int, int, const aiter_tensor_t*, cudaStream_t);
void launch_ep_dispatch(const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*, const aiter_tensor_t*,
                        const aiter_tensor_t*, int, int, int, const aiter_tensor_t*, cudaStream_t);
void ipc_export(const aiter_tensor_t*, void*, int64_t*);
void ipc_open(const void*, int, int64_t*);
void ipc_close(int64_t, int);

namespace {

// out = RNE(acc): 8 fp32 in, 8 half-precision values out per thread.
template <typename T2>
__global__ void __launch_bounds__(256) finalize_kernel(const float4* __restrict__ acc, uint4* __restrict__ out,
                                                       int64_t n8) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = __ldcs(acc + 2 * i), b = __ldcs(acc + 2 * i + 1);
        uint4 o;
        if constexpr (sizeof(T2) == sizeof(__nv_bfloat162) && std::is_same<T2, __nv_bfloat162>::value) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
            o = make_uint4(*(uint32_t*)&p0, *(uint32_t*)&p1, *(uint32_t*)&p2, *(uint32_t*)&p3);
        } else {
            __half2 p0 = __floats2half2_rn(a.x, a.y), p1 = __floats2half2_rn(a.z, a.w);
            __half2 p2 = __floats2half2_rn(b.x, b.y), p3 = __floats2half2_rn(b.z, b.w);
            o = make_uint4(*(uint32_t*)&p0, *(uint32_t*)&p1, *(uint32_t*)&p2, *(uint32_t*)&p3);
        }
        out[i] = o;
    }
}

void launch_finalize(aiter_tensor_t* out, const aiter_tensor_t* acc, cudaStream_t stream) {
    check_tensor(acc, "acc", AITER_DTYPE_fp32, -1);
    check_tensor(out, "out", -1, -1);
    B200_CHECK(out->dtype_ == AITER_DTYPE_bf16 || out->dtype_ == AITER_DTYPE_fp16,
               "out must be bf16 or fp16");
    B200_CHECK(out->numel_ == acc->numel_, "out and acc must have the same number of elements");
    B200_CHECK(acc->numel_ % 8 == 0, "element count must be a multiple of 8");
    B200_CHECK(((uintptr_t)acc->ptr & 15) == 0 && ((uintptr_t)out->ptr & 15) == 0, "buffers must be 16-byte aligned");
    const int64_t n8 = (int64_t)acc->numel_ / 8;
    if (n8 == 0) return;
    int64_t blocks = (n8 + 255) / 256;
    const int64_t cap = (int64_t)sm_count(acc->device_id) * 8;
    if (blocks > cap) blocks = cap;
    if (out->dtype_ == AITER_DTYPE_bf16)
        finalize_kernel<__nv_bfloat162><<<(unsigned)blocks, 256, 0, stream>>>((const float4*)acc->ptr, (uint4*)out->ptr, n8);
    else
        finalize_kernel<__half2><<<(unsigned)blocks, 256, 0, stream>>>((const float4*)acc->ptr, (uint4*)out->ptr, n8);
    B200_CUDA(cudaGetLastError());
}

}  // namespace
}  // namespace b200

using namespace b200;

#define B200_EXPORT __attribute__((visibility("default")))

extern "C" {

B200_EXPORT int aiter_ctypes_abi_version(void) { return 4; }

B200_EXPORT const char* aiter_get_last_error(void) { return last_error().empty() ? nullptr : last_error().c_str(); }

B200_EXPORT void aiter_clear_last_error(void) { last_error().clear(); }

B200_EXPORT int64_t b200_moe_sorting_get_workspace_size(int tokens, int num_experts, int topk, int dispatch_policy) {
    (void)dispatch_policy;  // the size covers both of this library's sort paths
    return sorting_workspace_bytes(tokens, num_experts, topk);
}

B200_EXPORT int b200_moe_sorting_fwd(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                         aiter_tensor_t* sorted_token_ids, aiter_tensor_t* sorted_weights,
                         aiter_tensor_t* sorted_expert_ids, aiter_tensor_t* num_valid_ids, aiter_tensor_t* moe_buf,
                         int num_experts, int unit_size, const aiter_tensor_t* local_expert_mask,
                         const aiter_tensor_t* num_local_tokens, aiter_tensor_t* workspace, int dispatch_policy,
                         aiter_tensor_t* local_topk_ids, aiter_tensor_t* m_indices, aiter_tensor_t* reverse_sorted,
                         void* stream) {
    (void)dispatch_policy;  // the reference's one-shot / multi-phase choice; made from the sizes here
    return safe_call([&] {
        B200_CHECK(topk_ids != nullptr, "topk_ids must not be NULL");
        B200_CHECK(m_indices == nullptr, "m_indices (per-row expert index of the grouped-GEMM layout) is not produced by "
                   "this library: pass NULL");
        B200_CHECK(reverse_sorted == nullptr, "reverse_sorted (token-slot to sorted-position map) is not produced by this "
                   "library: pass NULL");
        DeviceGuard g(topk_ids->device_id);
        launch_moe_sorting(topk_ids, topk_weights, sorted_token_ids, sorted_weights, sorted_expert_ids,
                           num_valid_ids, moe_buf, num_experts, unit_size, local_expert_mask, num_local_tokens,
                           workspace, local_topk_ids, (cudaStream_t)stream);
    });
}

// The sort for callers that cannot provide a workspace (see moe_sorting.cu): same outputs as
// b200_moe_sorting_fwd, scratch taken from a fixed array inside the library.  The first call on a
// device looks up the array's device address (cudaGetSymbolAddress) and should therefore happen
// before any stream capture; later calls only launch kernels.  All calls on one device share the
// array, so two of them must not overlap on the GPU (different streams without ordering would race).
B200_EXPORT int b200_moe_sorting_fwd_noalloc(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                                             aiter_tensor_t* sorted_token_ids, aiter_tensor_t* sorted_weights,
                                             aiter_tensor_t* sorted_expert_ids, aiter_tensor_t* num_valid_ids,
                                             aiter_tensor_t* moe_buf, int num_experts, int unit_size,
                                             const aiter_tensor_t* local_expert_mask,
                                             const aiter_tensor_t* num_local_tokens, aiter_tensor_t* local_topk_ids,
                                             void* stream) {
    return safe_call([&] {
        B200_CHECK(topk_ids != nullptr, "topk_ids must not be NULL");
        DeviceGuard g(topk_ids->device_id);
        launch_moe_sorting_noalloc(topk_ids, topk_weights, sorted_token_ids, sorted_weights, sorted_expert_ids,
                                   num_valid_ids, moe_buf, num_experts, unit_size, local_expert_mask,
                                   num_local_tokens, local_topk_ids, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_quant_1x128(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                                     const aiter_tensor_t* num_rows, int num_rows_factor, int transpose_scale, void* stream) {
    return safe_call([&] {
        B200_CHECK(input != nullptr, "input must not be NULL");
        DeviceGuard g(input->device_id);
        launch_quant_1x128(out, input, scales, num_rows, num_rows_factor, transpose_scale, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_quant_per_token(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scales,
                                         const aiter_tensor_t* num_rows, int num_rows_factor, void* stream) {
    return safe_call([&] {
        B200_CHECK(input != nullptr, "input must not be NULL");
        DeviceGuard g(input->device_id);
        launch_quant_per_token(out, input, scales, num_rows, num_rows_factor, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_stage1(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale, const aiter_tensor_t* w1,
                    const aiter_tensor_t* w1_scale, const aiter_tensor_t* sorted_token_ids,
                    const aiter_tensor_t* sorted_expert_ids, const aiter_tensor_t* num_valid_ids, aiter_tensor_t* a2,
                    aiter_tensor_t* a2_scale, aiter_tensor_t* status, int quant_type,
                    const aiter_tensor_t* sorted_weights, int activation, void* stream) {
    return safe_call([&] {
        B200_CHECK(a1 != nullptr, "a1 must not be NULL");
        DeviceGuard g(a1->device_id);
        launch_moe_stage1(a1, a1_scale, w1, w1_scale, sorted_token_ids, sorted_expert_ids, num_valid_ids, a2,
                          a2_scale, status, quant_type, sorted_weights, activation, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_stage2(const aiter_tensor_t* a2, const aiter_tensor_t* a2_scale, const aiter_tensor_t* w2,
                    const aiter_tensor_t* w2_scale, const aiter_tensor_t* sorted_token_ids,
                    const aiter_tensor_t* sorted_weights, const aiter_tensor_t* sorted_expert_ids,
                    const aiter_tensor_t* num_valid_ids, aiter_tensor_t* acc, aiter_tensor_t* status, int col_begin,
                    int col_end, int sm_margin, int quant_type, int doweight, void* stream) {
    return safe_call([&] {
        B200_CHECK(a2 != nullptr, "a2 must not be NULL");
        DeviceGuard g(a2->device_id);
        launch_moe_stage2(a2, a2_scale, w2, w2_scale, sorted_token_ids, sorted_weights, sorted_expert_ids,
                          num_valid_ids, acc, status, col_begin, col_end, sm_margin, quant_type, doweight, (cudaStream_t)stream);
    });
}

// Self-test of the bounded device-side waits: sets, for every later GEMM launch of this process, the wait limit in SM
// clocks (<= 0: the built-in ~2 s) and whether the weight producer loads nothing. With the producer stalled no copy or
// MMA is ever in flight, so the waits simply run out: every CTA winds down, frees its tensor memory and sets the
// caller's status word. Not for production use.
B200_EXPORT int b200_moe_debug_config(int64_t wait_limit_cycles, int stall_weight_producer) {
    return safe_call([&] { set_gemm_debug((long long)wait_limit_cycles, stall_weight_producer); });
}

B200_EXPORT int b200_biased_grouped_topk(const aiter_tensor_t* gating_output, const aiter_tensor_t* correction_bias,
                                         aiter_tensor_t* topk_weights, aiter_tensor_t* topk_ids, int num_expert_group,
                                         int topk_group, int need_renorm, float routed_scaling_factor, void* stream) {
    return safe_call([&] {
        B200_CHECK(gating_output != nullptr, "gating_output must not be NULL");
        DeviceGuard g(gating_output->device_id);
        launch_biased_grouped_topk(gating_output, correction_bias, topk_weights, topk_ids, num_expert_group, topk_group,
                                   need_renorm, routed_scaling_factor, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_topk_softmax(aiter_tensor_t* topk_weights, aiter_tensor_t* topk_indices,
                                  aiter_tensor_t* token_expert_indices, const aiter_tensor_t* gating_output,
                                  int need_renorm, void* stream) {
    return safe_call([&] {
        B200_CHECK(gating_output != nullptr, "gating_output must not be NULL");
        DeviceGuard g(gating_output->device_id);
        launch_topk_softmax(topk_weights, topk_indices, token_expert_indices, gating_output, need_renorm,
                            (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_finalize(aiter_tensor_t* out, const aiter_tensor_t* acc, void* stream) {
    return safe_call([&] {
        B200_CHECK(acc != nullptr, "acc must not be NULL");
        DeviceGuard g(acc->device_id);
        launch_finalize(out, acc, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_moe_quant_per_tensor(aiter_tensor_t* out, const aiter_tensor_t* input, aiter_tensor_t* scale,
                                          aiter_tensor_t* amax, aiter_tensor_t* row_scales,
                                          const aiter_tensor_t* row_limit, void* stream) {
    return safe_call([&] {
        B200_CHECK(input != nullptr, "input must not be NULL");
        DeviceGuard g(input->device_id);
        launch_quant_per_tensor(out, input, scale, amax, row_scales, row_limit, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_ep_dispatch(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale, const aiter_tensor_t* topk_ids,
                                 const aiter_tensor_t* peer_a1, const aiter_tensor_t* peer_a1_scale, int rank, int world,
                                 int experts_per_rank, const aiter_tensor_t* expert_rank, void* stream) {
    return safe_call([&] {
        B200_CHECK(a1 != nullptr, "a1 must not be NULL");
        DeviceGuard g(a1->device_id);
        launch_ep_dispatch(a1, a1_scale, topk_ids, peer_a1, peer_a1_scale, rank, world, experts_per_rank, expert_rank,
                           (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_ep_quant_dispatch(const aiter_tensor_t* input, const aiter_tensor_t* topk_ids, const aiter_tensor_t* peer_a1,
                                       const aiter_tensor_t* peer_a1_scale, int rank, int world, int experts_per_rank,
                                       const aiter_tensor_t* expert_rank, void* stream) {
    return safe_call([&] {
        B200_CHECK(input != nullptr, "input must not be NULL");
        DeviceGuard g(input->device_id);
        launch_ep_quant_dispatch(input, topk_ids, peer_a1, peer_a1_scale, rank, world, experts_per_rank, expert_rank,
                                 (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_ep_push_partials(const aiter_tensor_t* acc, const aiter_tensor_t* topk_ids,
                                      const aiter_tensor_t* peer_recv, int rank, int world, int experts_per_rank,
                                      const aiter_tensor_t* expert_rank, int col_begin, int col_end, int sm_limit,
                                      void* stream) {
    return safe_call([&] {
        B200_CHECK(acc != nullptr, "acc must not be NULL");
        DeviceGuard g(acc->device_id);
        launch_ep_push(acc, topk_ids, peer_recv, rank, world, experts_per_rank, expert_rank, col_begin, col_end, sm_limit,
                       (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_ep_combine(aiter_tensor_t* out, const aiter_tensor_t* acc, const aiter_tensor_t* recv,
                                const aiter_tensor_t* topk_ids, int rank, int world, int experts_per_rank,
                                const aiter_tensor_t* expert_rank, void* stream) {
    return safe_call([&] {
        B200_CHECK(acc != nullptr, "acc must not be NULL");
        DeviceGuard g(acc->device_id);
        launch_ep_combine(out, acc, recv, topk_ids, rank, world, experts_per_rank, expert_rank, (cudaStream_t)stream);
    });
}

B200_EXPORT int b200_ep_ipc_export(const aiter_tensor_t* tensor, void* handle_out, int64_t* offset_out) {
    return safe_call([&] { ipc_export(tensor, handle_out, offset_out); });
}

B200_EXPORT int b200_ep_ipc_open(const void* handle, int device, int64_t* ptr_out) {
    return safe_call([&] { ipc_open(handle, device, ptr_out); });
}

B200_EXPORT int b200_ep_ipc_close(int64_t ptr, int device) {
    return safe_call([&] { ipc_close(ptr, device); });
}

}  // extern "C"
