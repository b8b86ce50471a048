// Expert-parallel combine over NVLink peer memory: every rank pushes the fp32 partial rows it really
// produced to the rank that owns the token, the owner adds what arrived to its own partial.
//
// Takes the place of the dense fp32 reduce-scatter of the [M, H] partials: with group-limited routing a
// token has routes on at most half of 8 ranks, so half of the rows of a dense exchange are zeros. The
// reference reaches the same end with MoRI's combine, or with a stage-2 epilogue that scatters to an arena
// in peer memory (`Stage2ScatterContext`, aiter/fused_moe.py:536-575; oracle
// op_tests/multigpu_tests/test_dispatch_combine.py:18-72: the sum over ranks equals the single-GPU result).
//
// Protocol per layer call (all stream-ordered, no device-side waiting between ranks):
//   1. push kernel on rank r: for every token t of another owner o that has a route to one of r's experts,
//      copy acc_r[t, :] into recv_o[r, t - o*m_local, :] with 16-byte peer stores;
//   2. a collective of the communication library (any all-reduce) as the barrier: a rank passes it only
//      after every rank's push kernel has completed, i.e. after all peer stores are performed;
//   3. combine kernel on owner o: out[t] = round(sum over ranks r in ascending order of
//      (r == o ? acc_o[t] : recv_o[r, t_local]) for the ranks that touched t). A fixed order: the result
//      does not depend on arrival order.
// Whether rank r touched token t follows from the routing table alone (ids / experts_per_rank == r), which
// every rank holds after the all-gather, so no counts or indices are exchanged and rows that were not
// written are never read (recv needs no zero-fill).
//
// Plain peer loads/stores only: no multimem, no cluster launch.

#include <algorithm>
#include <cstring>

#include <cuda.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "quant_device.cuh"

namespace b200 {
namespace {

constexpr int kEpThreads = 256;
constexpr int kMaxWorld = 64;

// bit r set: token has a route to an expert of rank r
// expert_rank (optional): [global experts] owning rank of every expert, for placements that are not contiguous
// slices (a placement balanced by routing statistics); NULL = expert e lives on rank e / experts_per_rank.
__device__ __forceinline__ unsigned long long touch_mask(const int* __restrict__ ids, int topk, int experts_per_rank,
                                                         int world, const int* __restrict__ expert_rank) {
    unsigned long long m = 0;
    for (int k = 0; k < topk; ++k) {
        const int e = ids[k];
        if (e >= 0) {
            const int r = expert_rank ? __ldg(expert_rank + e) : e / experts_per_rank;
            if (r >= 0 && r < world) m |= 1ull << r;
        }
    }
    return m;
}

__global__ void __launch_bounds__(kEpThreads) ep_push_kernel(const float4* __restrict__ acc, const int* __restrict__ topk_ids,
                                                             const long long* __restrict__ peer_recv, int M, int H4,
                                                             int topk, int rank, int world, int experts_per_rank,
                                                             int m_local, const int* __restrict__ expert_rank, int c0, int c1) {
    // columns [c0, c1) of every row, in 16-byte units: a launch per column range lets the caller push a finished range
    // of stage 2 while the next one is computed
    for (int t = blockIdx.x; t < M; t += gridDim.x) {
        const int owner = t / m_local;
        if (owner == rank) continue;
        const unsigned long long m = touch_mask(topk_ids + (size_t)t * topk, topk, experts_per_rank, world, expert_rank);
        if (!((m >> rank) & 1ull)) continue;
        const float4* src = acc + (size_t)t * H4;
        float4* dst = reinterpret_cast<float4*>(peer_recv[owner]) + ((size_t)rank * m_local + (t - owner * m_local)) * H4;
        for (int i = c0 + threadIdx.x; i < c1; i += kEpThreads) dst[i] = src[i];
    }
    __threadfence_system();   // the peer stores are performed before this kernel counts as complete
}

// Dispatch: the quantised row of every local token (codes + block scales) goes to the ranks that hold one of its
// experts, this rank's own buffer included (its address is in the table like any other), at the token's global row.
__global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(const uint4* __restrict__ a1, const uint32_t* __restrict__ a1s,
                                                                 const int* __restrict__ topk_ids,
                                                                 const long long* __restrict__ peer_a1,
                                                                 const long long* __restrict__ peer_a1s, int m_local, int H16,
                                                                 int KB, int topk, int rank, int world, int experts_per_rank,
                                                                 const int* __restrict__ expert_rank) {
    for (int tl = blockIdx.x; tl < m_local; tl += gridDim.x) {
        const unsigned long long m = touch_mask(topk_ids + (size_t)tl * topk, topk, experts_per_rank, world, expert_rank);
        const size_t t = (size_t)rank * m_local + tl;
        for (int r = 0; r < world; ++r) {
            if (!((m >> r) & 1ull)) continue;
            uint4* dq = reinterpret_cast<uint4*>(peer_a1[r]) + t * H16;
            uint32_t* ds = reinterpret_cast<uint32_t*>(peer_a1s[r]) + t * KB;
            for (int i = threadIdx.x; i < H16; i += kEpThreads) dq[i] = a1[(size_t)tl * H16 + i];
            for (int i = threadIdx.x; i < KB; i += kEpThreads) ds[i] = a1s[(size_t)tl * KB + i];
        }
    }
    __threadfence_system();
}

// Quantise-and-dispatch in one kernel: the 1x128 quantisation of a local token row (same arithmetic as the plain
// quantiser, quant_device.cuh) whose codes and scales are stored straight into the arenas of the ranks that hold one
// of the token's experts; the quantised row never exists in this rank's own memory unless this rank is among them.
// One CTA per token, 16 lanes per 128-element group, 8-byte peer stores (a warp's 32 lanes write 256 contiguous
// bytes), the group's scale by its first lane.
template <bool F16>
__global__ void __launch_bounds__(kEpThreads) ep_quant_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ topk_ids,
                                                                       const long long* __restrict__ peer_a1,
                                                                       const long long* __restrict__ peer_a1s, int m_local, int KB,
                                                                       int topk, int rank, int world, int experts_per_rank,
                                                                       const int* __restrict__ expert_rank) {
    const int sub = threadIdx.x & 15;
    const int passes = (KB + kEpThreads / 16 - 1) / (kEpThreads / 16);   // the same trip count for every thread
    for (int tl = blockIdx.x; tl < m_local; tl += gridDim.x) {
        const unsigned long long m = touch_mask(topk_ids + (size_t)tl * topk, topk, experts_per_rank, world, expert_rank);
        const size_t t = (size_t)rank * m_local + tl;
        for (int i = 0; i < passes; ++i) {
            const int g = i * (kEpThreads / 16) + (threadIdx.x >> 4);
            const bool live = g < KB;
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (live) raw = __ldg(x + ((size_t)tl * KB + g) * 16 + sub);
            uint2 codes;
            const float scale = quant_group16<F16>(raw, codes);
            if (!live) continue;
            for (int r = 0; r < world; ++r) {
                if (!((m >> r) & 1ull)) continue;
                reinterpret_cast<uint2*>(peer_a1[r])[(t * KB + g) * 16 + sub] = codes;
                if (sub == 0) reinterpret_cast<float*>(peer_a1s[r])[t * KB + g] = scale;
            }
        }
    }
    __threadfence_system();
}

template <typename T2>
__device__ __forceinline__ T2 to_pair(float a, float b);
template <>
__device__ __forceinline__ __nv_bfloat162 to_pair<__nv_bfloat162>(float a, float b) { return __floats2bfloat162_rn(a, b); }
template <>
__device__ __forceinline__ __half2 to_pair<__half2>(float a, float b) { return __floats2half2_rn(a, b); }

template <typename T2>
__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(uint2* __restrict__ out, const float4* __restrict__ acc,
                                                                const float4* __restrict__ recv,
                                                                const int* __restrict__ topk_ids, int H4, int topk, int rank,
                                                                int world, int experts_per_rank, int m_local,
                                                                const int* __restrict__ expert_rank) {
    for (int tl = blockIdx.x; tl < m_local; tl += gridDim.x) {
        const int t = rank * m_local + tl;
        const unsigned long long m = touch_mask(topk_ids + (size_t)t * topk, topk, experts_per_rank, world, expert_rank);
        for (int i = threadIdx.x; i < H4; i += kEpThreads) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < world; ++r) {
                if (!((m >> r) & 1ull)) continue;
                const float4 v = (r == rank) ? acc[(size_t)t * H4 + i] : recv[((size_t)r * m_local + tl) * H4 + i];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            T2 lo = to_pair<T2>(s.x, s.y), hi = to_pair<T2>(s.z, s.w);
            out[(size_t)tl * H4 + i] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
    }
}

const int* rank_table(const aiter_tensor_t* expert_rank) {
    if (!expert_rank) return nullptr;
    check_tensor(expert_rank, "expert_rank", AITER_DTYPE_i32, 1);
    return (const int*)expert_rank->ptr;
}

void check_common(const aiter_tensor_t* acc, const aiter_tensor_t* topk_ids, int rank, int world, int experts_per_rank,
                  int64_t& M, int64_t& H, int64_t& topk, int64_t& m_local) {
    check_tensor(acc, "acc", AITER_DTYPE_fp32, 2);
    check_tensor(topk_ids, "topk_ids", AITER_DTYPE_i32, 2);
    M = acc->shape[0];
    H = acc->shape[1];
    topk = topk_ids->shape[1];
    B200_CHECK(topk_ids->shape[0] == M, "topk_ids must have one row per row of acc");
    B200_CHECK(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "bad rank/world: ", rank, "/", world);
    B200_CHECK(experts_per_rank >= 1, "experts_per_rank must be positive");
    B200_CHECK(M % world == 0, "token count ", M, " must be divisible by the world size ", world);
    B200_CHECK(H % 4 == 0 && ((uintptr_t)acc->ptr & 15) == 0, "rows must be 16-byte multiples and 16-byte aligned");
    m_local = M / world;
}

}  // namespace

void launch_ep_dispatch(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale, const aiter_tensor_t* topk_ids,
                        const aiter_tensor_t* peer_a1, const aiter_tensor_t* peer_a1_scale, int rank, int world,
                        int experts_per_rank, const aiter_tensor_t* expert_rank, cudaStream_t stream) {
    check_tensor(a1, "a1", AITER_DTYPE_fp8, 2);
    check_tensor(a1_scale, "a1_scale", AITER_DTYPE_fp32, 2);
    check_tensor(topk_ids, "topk_ids", AITER_DTYPE_i32, 2);
    check_tensor(peer_a1, "peer_a1", AITER_DTYPE_i64, 1);
    check_tensor(peer_a1_scale, "peer_a1_scale", AITER_DTYPE_i64, 1);
    const int64_t m_local = a1->shape[0], H = a1->shape[1], KB = a1_scale->shape[1];
    B200_CHECK(a1_scale->shape[0] == m_local && topk_ids->shape[0] == m_local, "a1_scale / topk_ids rows must match a1");
    B200_CHECK(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "bad rank/world: ", rank, "/", world);
    B200_CHECK(experts_per_rank >= 1, "experts_per_rank must be positive");
    B200_CHECK((int64_t)peer_a1->numel_ == world && (int64_t)peer_a1_scale->numel_ == world,
               "peer tables need one address per rank");
    B200_CHECK(H % 16 == 0 && ((uintptr_t)a1->ptr & 15) == 0, "rows must be 16-byte multiples and 16-byte aligned");
    if (m_local == 0) return;
    const int grid = (int)std::min<int64_t>(m_local, (int64_t)sm_count(a1->device_id) * 8);
    ep_dispatch_kernel<<<grid, kEpThreads, 0, stream>>>((const uint4*)a1->ptr, (const uint32_t*)a1_scale->ptr,
                                                       (const int*)topk_ids->ptr, (const long long*)peer_a1->ptr,
                                                       (const long long*)peer_a1_scale->ptr, (int)m_local, (int)(H / 16),
                                                       (int)KB, (int)topk_ids->shape[1], rank, world, experts_per_rank,
                                                       rank_table(expert_rank));
    B200_CUDA(cudaGetLastError());
}

void launch_ep_quant_dispatch(const aiter_tensor_t* x, const aiter_tensor_t* topk_ids, const aiter_tensor_t* peer_a1,
                              const aiter_tensor_t* peer_a1_scale, int rank, int world, int experts_per_rank,
                              const aiter_tensor_t* expert_rank, cudaStream_t stream) {
    check_tensor(x, "input", -1, 2);
    B200_CHECK(x->dtype_ == AITER_DTYPE_bf16 || x->dtype_ == AITER_DTYPE_fp16, "input must be bf16 or fp16");
    check_tensor(topk_ids, "topk_ids", AITER_DTYPE_i32, 2);
    check_tensor(peer_a1, "peer_a1", AITER_DTYPE_i64, 1);
    check_tensor(peer_a1_scale, "peer_a1_scale", AITER_DTYPE_i64, 1);
    const int64_t m_local = x->shape[0], H = x->shape[1];
    B200_CHECK(topk_ids->shape[0] == m_local, "topk_ids rows must match the input");
    B200_CHECK(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "bad rank/world: ", rank, "/", world);
    B200_CHECK(experts_per_rank >= 1, "experts_per_rank must be positive");
    B200_CHECK((int64_t)peer_a1->numel_ == world && (int64_t)peer_a1_scale->numel_ == world,
               "peer tables need one address per rank");
    B200_CHECK(H % 128 == 0 && ((uintptr_t)x->ptr & 15) == 0, "rows must be multiples of 128 elements and 16-byte aligned");
    if (m_local == 0) return;
    const int grid = (int)std::min<int64_t>(m_local, (int64_t)sm_count(x->device_id) * 8);
    auto kern = x->dtype_ == AITER_DTYPE_fp16 ? ep_quant_dispatch_kernel<true> : ep_quant_dispatch_kernel<false>;
    kern<<<grid, kEpThreads, 0, stream>>>((const uint4*)x->ptr, (const int*)topk_ids->ptr, (const long long*)peer_a1->ptr,
                                          (const long long*)peer_a1_scale->ptr, (int)m_local, (int)(H / 128),
                                          (int)topk_ids->shape[1], rank, world, experts_per_rank, rank_table(expert_rank));
    B200_CUDA(cudaGetLastError());
}

void launch_ep_push(const aiter_tensor_t* acc, const aiter_tensor_t* topk_ids, const aiter_tensor_t* peer_recv, int rank,
                    int world, int experts_per_rank, const aiter_tensor_t* expert_rank, int col_begin, int col_end,
                    int sm_limit, cudaStream_t stream) {
    int64_t M, H, topk, m_local;
    check_common(acc, topk_ids, rank, world, experts_per_rank, M, H, topk, m_local);
    check_tensor(peer_recv, "peer_recv", AITER_DTYPE_i64, 1);
    B200_CHECK((int64_t)peer_recv->numel_ == world, "peer_recv needs one address per rank");
    if (col_end <= 0) col_end = (int)H;
    B200_CHECK(col_begin >= 0 && col_begin < col_end && col_end <= H && col_begin % 4 == 0 && col_end % 4 == 0,
               "column range [", col_begin, ", ", col_end, ") must lie in [0, model_dim] on 4-column boundaries");
    B200_CHECK(sm_limit >= 0, "sm_limit must not be negative");
    if (M == 0 || world == 1) return;
    // sm_limit > 0: at most that many SMs' worth of CTAs (8 per SM), for a push that runs beside a GEMM kernel on the
    // SMs the GEMM leaves free
    const int sms = sm_limit > 0 ? std::min(sm_limit, sm_count(acc->device_id)) : sm_count(acc->device_id);
    const int grid = (int)std::min<int64_t>(M, (int64_t)sms * 8);
    ep_push_kernel<<<grid, kEpThreads, 0, stream>>>((const float4*)acc->ptr, (const int*)topk_ids->ptr,
                                                   (const long long*)peer_recv->ptr, (int)M, (int)(H / 4), (int)topk, rank,
                                                   world, experts_per_rank, (int)m_local, rank_table(expert_rank),
                                                   col_begin / 4, col_end / 4);
    B200_CUDA(cudaGetLastError());
}

void launch_ep_combine(aiter_tensor_t* out, const aiter_tensor_t* acc, const aiter_tensor_t* recv,
                       const aiter_tensor_t* topk_ids, int rank, int world, int experts_per_rank,
                       const aiter_tensor_t* expert_rank, cudaStream_t stream) {
    int64_t M, H, topk, m_local;
    check_common(acc, topk_ids, rank, world, experts_per_rank, M, H, topk, m_local);
    check_tensor(out, "out", -1, 2);
    B200_CHECK(out->dtype_ == AITER_DTYPE_bf16 || out->dtype_ == AITER_DTYPE_fp16, "out must be bf16 or fp16");
    B200_CHECK(out->shape[0] == m_local && out->shape[1] == H, "out must be [tokens / world, model_dim]");
    check_tensor(recv, "recv", AITER_DTYPE_fp32, 3);
    B200_CHECK(recv->shape[0] == world && recv->shape[1] == m_local && recv->shape[2] == H,
               "recv must be [world, tokens / world, model_dim]");
    B200_CHECK(((uintptr_t)recv->ptr & 15) == 0 && ((uintptr_t)out->ptr & 7) == 0, "recv/out alignment");
    if (m_local == 0) return;
    const int grid = (int)std::min<int64_t>(m_local, (int64_t)sm_count(acc->device_id) * 8);
    if (out->dtype_ == AITER_DTYPE_bf16)
        ep_combine_kernel<__nv_bfloat162><<<grid, kEpThreads, 0, stream>>>(
            (uint2*)out->ptr, (const float4*)acc->ptr, (const float4*)recv->ptr, (const int*)topk_ids->ptr, (int)(H / 4),
            (int)topk, rank, world, experts_per_rank, (int)m_local, rank_table(expert_rank));
    else
        ep_combine_kernel<__half2><<<grid, kEpThreads, 0, stream>>>(
            (uint2*)out->ptr, (const float4*)acc->ptr, (const float4*)recv->ptr, (const int*)topk_ids->ptr, (int)(H / 4),
            (int)topk, rank, world, experts_per_rank, (int)m_local, rank_table(expert_rank));
    B200_CUDA(cudaGetLastError());
}

// ---- mapping another process's receive buffer (CUDA IPC) --------------------------------------------------------
// A mapping belongs to the device that was current when it was opened: a pointer opened under GPU b is not
// usable by kernels of GPU a, even with peer access enabled between the two. Every rank therefore opens its
// peers' handles with ITS OWN device current (cudaIpcMemLazyEnablePeerAccess sets up the peer mapping).

// handle_out: 64 bytes (cudaIpcMemHandle_t) for the allocation that holds t; offset_out: t's byte offset in it.
void ipc_export(const aiter_tensor_t* t, void* handle_out, int64_t* offset_out) {
    check_tensor(t, "tensor", -1, -1);
    B200_CHECK(handle_out != nullptr && offset_out != nullptr, "handle_out / offset_out must not be NULL");
    B200_CHECK(t->ptr != nullptr, "tensor has no storage");
    DeviceGuard guard(t->device_id);
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range_fn = nullptr;
    if (!range_fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        B200_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qres));
        B200_CHECK(sym != nullptr && qres == cudaDriverEntryPointSuccess, "cuMemGetAddressRange is not available");
        range_fn = reinterpret_cast<RangeFn>(sym);
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    CUresult r = range_fn(&base, &size, (CUdeviceptr)(uintptr_t)t->ptr);
    B200_CHECK(r == CUDA_SUCCESS, "cuMemGetAddressRange failed with code ", (int)r);
    cudaIpcMemHandle_t h;
    B200_CUDA(cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base));
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(handle_out, &h, sizeof(h));
    *offset_out = (int64_t)((uintptr_t)t->ptr - (uintptr_t)base);
}

// Opens a handle made by ipc_export in another process, for kernels of `device`.
void ipc_open(const void* handle, int device, int64_t* ptr_out) {
    B200_CHECK(handle != nullptr && ptr_out != nullptr, "handle / ptr_out must not be NULL");
    DeviceGuard guard(device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    B200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    B200_CHECK(p != nullptr, "cudaIpcOpenMemHandle returned a null pointer");
    cudaPointerAttributes attr;
    B200_CUDA(cudaPointerGetAttributes(&attr, p));
    B200_CHECK(attr.type == cudaMemoryTypeDevice, "the mapped pointer is not device memory (type ", (int)attr.type, ")");
    *ptr_out = (int64_t)(uintptr_t)p;
}

void ipc_close(int64_t ptr, int device) {
    DeviceGuard guard(device);
    B200_CUDA(cudaIpcCloseMemHandle((void*)(uintptr_t)ptr));
}

}  // namespace b200
