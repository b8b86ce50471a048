// Router kernels that feed moe_sorting / fused_moe: one warp per token, scores in registers.
//
//   biased_grouped_topk  DeepSeek-V3 style: sigmoid scores, + correction bias for the choice, groups ranked
//                        by the sum of their two best biased scores, top groups kept, top-k experts among
//                        them, weights = un-biased scores, renormalised, times routed_scaling_factor.
//                        Arithmetic of aiter/ops/topk.py:217-259 (biased_grouped_topk_torch); replaces the
//                        native op of aiter/ops/topk.py:89-99 / csrc/kernels/topk_softmax_kernels_group.cu:1219-1266.
//   topk_softmax         fp32 softmax, top-k, optional renormalisation (aiter/fused_moe.py:4058-4129,
//                        csrc/kernels/topk_softmax_kernels.cu:769).
//
// Expert e sits in lane e % 32, register e / 32.  Selections are repeated warp arg-max reductions
// (value, then lower index on ties), so the result does not depend on scheduling.

#include <cuda_bf16.h>
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarpsPerBlock = 8;
#define kNegInf (-CUDART_INF_F)

template <typename T>
__device__ __forceinline__ float load_f(const T* p, int64_t i);
template <>
__device__ __forceinline__ float load_f<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float load_f<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
    return __bfloat162float(p[i]);
}

// warp arg-max over (value, index): larger value wins, lower index on ties. All lanes get the result.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, d);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, d);
        if (ov > v || (ov == v && oi < idx)) {
            v = ov;
            idx = oi;
        }
    }
}

// Picks the k best of val[] (expert e = j*32 + lane) one at a time; lane i < k keeps pick i in (my_id, my_w),
// where the weight is taken from wsrc[] of the winning expert. Returns the sum of the k weights.
template <int VPL>
__device__ __forceinline__ float select_topk(float (&val)[VPL], const float (&wsrc)[VPL], int k, int lane,
                                             int& my_id, float& my_w) {
    float wsum = 0.f;
    for (int i = 0; i < k; ++i) {
        float best = kNegInf;
        int bidx = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int e = j * 32 + lane;
            if (val[j] > best || (val[j] == best && e < bidx)) {
                best = val[j];
                bidx = e;
            }
        }
        warp_argmax(best, bidx);
        // the owner of the winner publishes its weight and retires the entry
        float w = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            if (j * 32 + lane == bidx) {
                w = wsrc[j];
                val[j] = kNegInf;
            }
        }
        w = __shfl_sync(0xffffffffu, w, bidx & 31);
        wsum += w;
        if (lane == i) {
            my_id = bidx;
            my_w = w;
        }
    }
    return wsum;
}

template <typename TG, typename TB, int VPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) biased_grouped_topk_kernel(
    const TG* __restrict__ gating, const TB* __restrict__ bias, float* __restrict__ out_w, int* __restrict__ out_id,
    int tokens, int E, int topk, int n_group, int topk_group, int renorm, float scale) {
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const int gsize = E / n_group;
    float score[VPL], choice[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int e = j * 32 + lane;
        if (e < E) {
            const float x = load_f<TG>(gating, (int64_t)token * E + e);
            score[j] = __fdiv_rn(1.0f, 1.0f + expf(-x));
            choice[j] = score[j] + load_f<TB>(bias, e);
        } else {
            score[j] = 0.f;
            choice[j] = kNegInf;
        }
    }
    // group score = sum of the two largest biased scores of the group
    unsigned keep = 0;   // bit g: group g is kept (n_group <= 32)
    float gscore_mine = kNegInf;   // lane g holds the score of group g
    for (int g = 0; g < n_group; ++g) {
        float b1 = kNegInf;
        int i1 = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int e = j * 32 + lane;
            if (e < E && e / gsize == g && (choice[j] > b1 || (choice[j] == b1 && e < i1))) {
                b1 = choice[j];
                i1 = e;
            }
        }
        warp_argmax(b1, i1);
        float b2 = kNegInf;
        int i2 = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int e = j * 32 + lane;
            if (e < E && e / gsize == g && e != i1 && (choice[j] > b2 || (choice[j] == b2 && e < i2))) {
                b2 = choice[j];
                i2 = e;
            }
        }
        warp_argmax(b2, i2);
        const float gs = (gsize >= 2) ? b1 + b2 : b1;
        if (lane == g) gscore_mine = gs;
    }
    for (int i = 0; i < topk_group; ++i) {
        float v = (lane < n_group && !((keep >> lane) & 1u)) ? gscore_mine : kNegInf;
        int idx = lane;
        warp_argmax(v, idx);
        keep |= 1u << idx;
    }
    // experts of dropped groups compete with the value 0.0, as masked_fill(~mask, 0.0) does
    float cand[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int e = j * 32 + lane;
        cand[j] = (e < E) ? (((keep >> (e / gsize)) & 1u) ? choice[j] : 0.0f) : kNegInf;
    }
    int my_id = 0;
    float my_w = 0.f;
    const float wsum = select_topk<VPL>(cand, score, topk, lane, my_id, my_w);
    if (lane < topk) {
        float w = renorm ? __fdiv_rn(my_w, wsum) : my_w;
        out_w[(int64_t)token * topk + lane] = w * scale;
        out_id[(int64_t)token * topk + lane] = my_id;
    }
}

template <typename TG, int VPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) topk_softmax_kernel(
    const TG* __restrict__ gating, float* __restrict__ out_w, int* __restrict__ out_id, int* __restrict__ src_row,
    int tokens, int E, int topk, int renorm) {
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (token >= tokens) return;
    float x[VPL], prob[VPL];
    float mx = kNegInf;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int e = j * 32 + lane;
        x[j] = (e < E) ? load_f<TG>(gating, (int64_t)token * E + e) : kNegInf;
        mx = fmaxf(mx, x[j]);
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        prob[j] = (j * 32 + lane < E) ? expf(x[j] - mx) : 0.f;
        sum += prob[j];
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        prob[j] = __fdiv_rn(prob[j], sum);
        x[j] = (j * 32 + lane < E) ? prob[j] : kNegInf;   // selection keys
    }
    int my_id = 0;
    float my_w = 0.f;
    const float wsum = select_topk<VPL>(x, prob, topk, lane, my_id, my_w);
    if (lane < topk) {
        out_w[(int64_t)token * topk + lane] = renorm ? __fdiv_rn(my_w, wsum) : my_w;
        out_id[(int64_t)token * topk + lane] = my_id;
        if (src_row) src_row[(int64_t)token * topk + lane] = lane * tokens + token;
    }
}

template <typename F>
void dispatch_vpl(int E, F&& f) {
    const int need = (E + 31) / 32;
    if (need <= 1) f(std::integral_constant<int, 1>{});
    else if (need <= 2) f(std::integral_constant<int, 2>{});
    else if (need <= 4) f(std::integral_constant<int, 4>{});
    else if (need <= 8) f(std::integral_constant<int, 8>{});
    else if (need <= 16) f(std::integral_constant<int, 16>{});
    else f(std::integral_constant<int, 32>{});
}

void check_outputs(const aiter_tensor_t* gating, const aiter_tensor_t* w, const aiter_tensor_t* ids, int64_t& tokens,
                   int64_t& E, int64_t& topk) {
    check_tensor(gating, "gating_output", -1, 2);
    B200_CHECK(gating->dtype_ == AITER_DTYPE_fp32 || gating->dtype_ == AITER_DTYPE_bf16,
               "gating_output must be fp32 or bf16");
    check_tensor(w, "topk_weights", AITER_DTYPE_fp32, 2);
    check_tensor(ids, "topk_ids", AITER_DTYPE_i32, 2);
    tokens = gating->shape[0];
    E = gating->shape[1];
    topk = ids->shape[1];
    B200_CHECK(E >= 1 && E <= 1024, "number of experts must be in [1, 1024], got ", E);
    B200_CHECK(topk >= 1 && topk <= 32 && topk <= E, "topk must be in [1, min(32, experts)], got ", topk);
    B200_CHECK(w->shape[0] >= tokens && ids->shape[0] >= tokens && w->shape[1] == topk,
               "topk_weights / topk_ids must be [tokens, topk]");
}

}  // namespace

void launch_biased_grouped_topk(const aiter_tensor_t* gating, const aiter_tensor_t* bias, aiter_tensor_t* w,
                                aiter_tensor_t* ids, int n_group, int topk_group, int renorm, float scale,
                                cudaStream_t stream) {
    int64_t tokens, E, topk;
    check_outputs(gating, w, ids, tokens, E, topk);
    check_tensor(bias, "correction_bias", -1, 1);
    B200_CHECK(bias->dtype_ == AITER_DTYPE_fp32 || bias->dtype_ == AITER_DTYPE_bf16, "correction_bias must be fp32 or bf16");
    B200_CHECK((int64_t)bias->numel_ == E, "correction_bias must have one entry per expert");
    B200_CHECK(n_group >= 1 && n_group <= 32 && E % n_group == 0, "num_expert_group must divide the expert count and be <= 32");
    B200_CHECK(topk_group >= 1 && topk_group <= n_group, "topk_group must be in [1, num_expert_group]");
    if (tokens == 0) return;
    const unsigned grid = (unsigned)((tokens + kWarpsPerBlock - 1) / kWarpsPerBlock);
    dispatch_vpl((int)E, [&](auto vpl) {
        constexpr int V = decltype(vpl)::value;
        auto go = [&](auto* g, auto* b) {
            using TG = std::remove_cv_t<std::remove_pointer_t<decltype(g)>>;
            using TB = std::remove_cv_t<std::remove_pointer_t<decltype(b)>>;
            biased_grouped_topk_kernel<TG, TB, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
                g, b, (float*)w->ptr, (int*)ids->ptr, (int)tokens, (int)E, (int)topk, n_group, topk_group, renorm, scale);
        };
        const bool gf = gating->dtype_ == AITER_DTYPE_fp32, bf = bias->dtype_ == AITER_DTYPE_fp32;
        if (gf && bf) go((const float*)gating->ptr, (const float*)bias->ptr);
        else if (gf) go((const float*)gating->ptr, (const __nv_bfloat16*)bias->ptr);
        else if (bf) go((const __nv_bfloat16*)gating->ptr, (const float*)bias->ptr);
        else go((const __nv_bfloat16*)gating->ptr, (const __nv_bfloat16*)bias->ptr);
    });
    B200_CUDA(cudaGetLastError());
}

void launch_topk_softmax(aiter_tensor_t* w, aiter_tensor_t* ids, aiter_tensor_t* src_row, const aiter_tensor_t* gating,
                         int renorm, cudaStream_t stream) {
    int64_t tokens, E, topk;
    check_outputs(gating, w, ids, tokens, E, topk);
    if (src_row) {
        check_tensor(src_row, "token_expert_indices", AITER_DTYPE_i32, 2);
        B200_CHECK(src_row->shape[0] >= tokens && src_row->shape[1] == topk, "token_expert_indices must be [tokens, topk]");
    }
    if (tokens == 0) return;
    const unsigned grid = (unsigned)((tokens + kWarpsPerBlock - 1) / kWarpsPerBlock);
    dispatch_vpl((int)E, [&](auto vpl) {
        constexpr int V = decltype(vpl)::value;
        if (gating->dtype_ == AITER_DTYPE_fp32)
            topk_softmax_kernel<float, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
                (const float*)gating->ptr, (float*)w->ptr, (int*)ids->ptr, src_row ? (int*)src_row->ptr : nullptr,
                (int)tokens, (int)E, (int)topk, renorm);
        else
            topk_softmax_kernel<__nv_bfloat16, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
                (const __nv_bfloat16*)gating->ptr, (float*)w->ptr, (int*)ids->ptr, src_row ? (int*)src_row->ptr : nullptr,
                (int)tokens, (int)E, (int)topk, renorm);
    });
    B200_CUDA(cudaGetLastError());
}

}  // namespace b200
