// moe_sorting for sm_100a: stable counting sort of (token, slot) routes by expert, every
// expert padded to a multiple of unit_size.  Output contract of the reference's native sort
// (csrc/include/moe_sorting_opus.h:280-359) with the padding values of its torch oracle
// (op_tests/test_moe_sorting.py:45-99).
//
// Route r = token*topk + slot.  Within an expert routes keep ascending r, which is the order
// torch.where() yields in the oracle.  Each warp owns a contiguous run of routes, so the
// position of a route is
//     base[expert] + (routes of that expert in earlier CTAs) + (in earlier warps of this CTA)
//                  + (in earlier 32-route steps of this warp) + (in lower lanes of this step)
// where the last term comes from __match_any_sync + popc.  No atomics on the output side:
// the result is deterministic.
//
// Two launch shapes:
//   single CTA   routes <= kSingleMaxRoutes: count, scan, fill and scatter in one kernel;
//   multi CTA    count per 4096-route chunk -> scan (1 CTA) -> scatter per chunk, with the
//                per-chunk counts and expert bases in a caller-provided workspace.
// Extra CTAs zero-fill moe_buf when the caller passes one (in the single kernel, or beside the scan).

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 4096;            // routes per CTA on the multi-CTA path
constexpr int kSingleMaxRoutes = 16384; // above this the multi-CTA path is used
constexpr int kMaxExperts = 1024;

struct SortArgs {
    const int* ids;
    const float* weights;
    const int* mask;       // [E] or null
    const int* num_local;  // [1] or null
    int* sorted_ids;
    float* sorted_w;
    int* sorted_eids;
    int* num_valid;
    int* local_topk_ids;   // [M*topk] or null
    int* ws_cnt;           // [nchunks*E]   (multi-CTA only)
    int* ws_base;          // [E]           (multi-CTA only)
    uint4* zero_buf;       // moe_buf or null
    size_t zero_vec16;     // number of 16-byte words to clear
    unsigned char* zero_tail;
    int zero_tail_bytes;
    int M, topk, E, unit;
    int max_padded, max_blocks;
    int nchunks;           // CTAs that sort (1 on the single-CTA path)
};

__device__ __forceinline__ int eff_tokens(const SortArgs& a) {
    int t = a.M;
    if (a.num_local) {
        int v = *a.num_local;
        v = v < 0 ? 0 : v;
        t = v < t ? v : t;
    }
    return t;
}

// Exclusive scan of one int per thread over the whole CTA (kThreads threads).
__device__ __forceinline__ int block_scan_excl(int v, int* warp_tot, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int t = warp_tot[lane];
        int ti = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, ti, d);
            if (lane >= d) ti += n;
        }
        warp_tot[lane] = ti - t;  // exclusive prefix of warp totals
        if (lane == 31) warp_tot[32] = ti;
    }
    __syncthreads();
    total = warp_tot[32];
    int r = warp_tot[warp] + incl - v;
    __syncthreads();
    return r;
}

__device__ __forceinline__ void zero_fill(const SortArgs& a, int part, int nparts) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (size_t i = (size_t)part * kThreads + threadIdx.x; i < a.zero_vec16;
         i += (size_t)nparts * kThreads)
        a.zero_buf[i] = z;
    if (part == 0 && (int)threadIdx.x < a.zero_tail_bytes) a.zero_tail[threadIdx.x] = 0;
}

// local_id[e] = cumsum(mask)-1 for kept experts, -1 for dropped ones.
__device__ __forceinline__ void build_local_ids(const SortArgs& a, int* local_id, int* warp_tot) {
    const int e = threadIdx.x;
    int keep = (e < a.E) ? (a.mask ? (a.mask[e] != 0) : 1) : 0;
    int total;
    int excl = block_scan_excl(keep, warp_tot, total);
    if (e < a.E) local_id[e] = keep ? excl : -1;
    __syncthreads();
}

// Per-warp histogram of routes [r0, r1): hist[w*E + e].  Warp w owns
// [r0 + w*seg, r0 + (w+1)*seg) with seg a multiple of 32.
__device__ __forceinline__ int warp_segment(int r0, int r1) {
    int n = r1 - r0;
    int seg = (n + kWarps - 1) / kWarps;
    return (seg + 31) & ~31;
}

__device__ __forceinline__ void count_routes(const SortArgs& a, int* hist, int r0, int r1) {
    for (int i = threadIdx.x; i < kWarps * a.E; i += kThreads) hist[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = warp_segment(r0, r1);
    const int s0 = r0 + warp * seg;
    const int s1 = min(s0 + seg, r1);
    for (int i = s0 + lane; i < s1; i += 32) {
        int e = a.ids[i];
        if (e >= 0 && e < a.E) atomicAdd(&hist[warp * a.E + e], 1);
    }
    __syncthreads();
}

// hist[w][e] -> exclusive prefix over w; returns the CTA total for expert e = threadIdx.x.
__device__ __forceinline__ int prefix_over_warps(const SortArgs& a, int* hist) {
    int run = 0;
    const int e = threadIdx.x;
    if (e < a.E) {
#pragma unroll 4
        for (int w = 0; w < kWarps; ++w) {
            int c = hist[w * a.E + e];
            hist[w * a.E + e] = run;
            run += c;
        }
    }
    return run;
}

__device__ __forceinline__ void scatter_routes(const SortArgs& a, int* hist, const int* gbase,
                                               const int* local_id, int r0, int r1) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = warp_segment(r0, r1);
    const int s0 = r0 + warp * seg;
    const int s1 = min(s0 + seg, r1);
    const unsigned lt = (1u << lane) - 1u;
    for (int it = s0; it < s1; it += 32) {
        const int i = it + lane;
        const bool in = i < s1;
        int e = in ? a.ids[i] : -1;
        int lid = (in && e >= 0 && e < a.E) ? local_id[e] : -1;
        const bool live = in && e >= 0 && e < a.E;
        // lanes with the same expert form a group; others get a private key
        unsigned grp = __match_any_sync(0xffffffffu, live ? e : (a.E + lane));
        int rank = __popc(grp & lt);
        int off = live ? hist[warp * a.E + e] : 0;
        __syncwarp();
        if (live && rank == 0) hist[warp * a.E + e] = off + __popc(grp);
        __syncwarp();
        if (in && a.local_topk_ids) a.local_topk_ids[i] = lid;
        if (lid >= 0) {
            int pos = gbase[e] + off + rank;
            int token = i / a.topk;
            int slot = i - token * a.topk;
            a.sorted_ids[pos] = (slot << 24) | token;
            a.sorted_w[pos] = a.weights[i];
        }
    }
}

// Given cnt (routes of expert e) writes: base[e] (smem), expert ids of its blocks, its pad
// entries, the tail past the padded total, num_valid.
__device__ __forceinline__ void layout_experts(const SortArgs& a, int cnt, const int* local_id,
                                               int* base, int* warp_tot, int tokens) {
    const int e = threadIdx.x;
    int lid = (e < a.E) ? local_id[e] : -1;
    int padded = (lid >= 0 && cnt > 0) ? ((cnt + a.unit - 1) / a.unit) * a.unit : 0;
    int total;
    int b = block_scan_excl(padded, warp_tot, total);
    if (e < a.E) base[e] = b;
    const int pad_id = (a.topk << 24) | a.M;
    if (padded > 0) {
        for (int k = 0; k < padded / a.unit; ++k) a.sorted_eids[b / a.unit + k] = lid;
        for (int p = b + cnt; p < b + padded; ++p) {
            a.sorted_ids[p] = pad_id;
            a.sorted_w[p] = 0.f;
        }
    }
    for (int k = total / a.unit + threadIdx.x; k < a.max_blocks; k += kThreads) a.sorted_eids[k] = -1;
    for (int p = total + threadIdx.x; p < a.max_padded; p += kThreads) {
        a.sorted_ids[p] = pad_id;
        a.sorted_w[p] = 0.f;
    }
    if (threadIdx.x == 0) {
        a.num_valid[0] = total;
        a.num_valid[1] = tokens;
    }
    __syncthreads();
}

__device__ __forceinline__ void clear_unsorted_local_ids(const SortArgs& a, int routes, int part,
                                                         int nparts) {
    if (!a.local_topk_ids) return;
    for (int i = routes + part * kThreads + threadIdx.x; i < a.M * a.topk; i += nparts * kThreads)
        a.local_topk_ids[i] = -1;
}

extern __shared__ int smem_i[];
// smem: hist[kWarps*E] | local_id[E] | base[E] | warp_tot[40]

__global__ void __launch_bounds__(kThreads, 1) sort_single_kernel(SortArgs a) {
    if ((int)blockIdx.x >= a.nchunks) {
        zero_fill(a, blockIdx.x - a.nchunks, gridDim.x - a.nchunks);
        return;
    }
    int* hist = smem_i;
    int* local_id = hist + kWarps * a.E;
    int* base = local_id + a.E;
    int* warp_tot = base + a.E;
    const int tokens = eff_tokens(a);
    const int routes = tokens * a.topk;
    build_local_ids(a, local_id, warp_tot);
    count_routes(a, hist, 0, routes);
    int cnt = prefix_over_warps(a, hist);
    layout_experts(a, cnt, local_id, base, warp_tot, tokens);
    scatter_routes(a, hist, base, local_id, 0, routes);
    clear_unsorted_local_ids(a, routes, 0, 1);
}

__global__ void __launch_bounds__(kThreads, 1) sort_count_kernel(SortArgs a) {
    int* hist = smem_i;
    const int routes = eff_tokens(a) * a.topk;
    const int r0 = min((int)blockIdx.x * kChunk, routes);
    const int r1 = min(r0 + kChunk, routes);
    count_routes(a, hist, r0, r1);
    int cnt = prefix_over_warps(a, hist);
    if ((int)threadIdx.x < a.E) a.ws_cnt[blockIdx.x * a.E + threadIdx.x] = cnt;
}

__global__ void __launch_bounds__(kThreads, 1) sort_scan_kernel(SortArgs a) {
    // CTA 0 scans; the others zero-fill moe_buf beside it. The scan is one CTA's worth of latency (tens of
    // microseconds at 64 K routes), the fill is bandwidth: in the same launch the fill costs nothing extra, in the
    // count kernel (which is over in microseconds) it would delay the two kernels behind it by its whole length.
    if (blockIdx.x >= 1) {
        zero_fill(a, blockIdx.x - 1, gridDim.x - 1);
        return;
    }
    int* local_id = smem_i;
    int* base = local_id + a.E;
    int* warp_tot = base + a.E;
    const int tokens = eff_tokens(a);
    build_local_ids(a, local_id, warp_tot);
    int run = 0;
    const int e = threadIdx.x;
    if (e < a.E) {
        // 8 independent loads in flight at a time (the stores in between would otherwise serialise them)
        for (int c0 = 0; c0 < a.nchunks; c0 += 8) {
            int v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = (c0 + k < a.nchunks) ? __ldcg(a.ws_cnt + (c0 + k) * a.E + e) : 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (c0 + k < a.nchunks) a.ws_cnt[(c0 + k) * a.E + e] = run;  // routes of e in earlier chunks
                run += v[k];
            }
        }
    }
    layout_experts(a, run, local_id, base, warp_tot, tokens);
    if (e < a.E) a.ws_base[e] = base[e];
}

__global__ void __launch_bounds__(kThreads, 1) sort_scatter_kernel(SortArgs a) {
    int* hist = smem_i;
    int* local_id = hist + kWarps * a.E;
    int* base = local_id + a.E;
    int* warp_tot = base + a.E;
    const int routes = eff_tokens(a) * a.topk;
    const int r0 = min((int)blockIdx.x * kChunk, routes);
    const int r1 = min(r0 + kChunk, routes);
    build_local_ids(a, local_id, warp_tot);
    count_routes(a, hist, r0, r1);
    prefix_over_warps(a, hist);
    if ((int)threadIdx.x < a.E)
        base[threadIdx.x] = a.ws_base[threadIdx.x] + a.ws_cnt[blockIdx.x * a.E + threadIdx.x];
    __syncthreads();
    scatter_routes(a, hist, base, local_id, r0, r1);
    clear_unsorted_local_ids(a, routes, blockIdx.x, gridDim.x);
}

inline int num_chunks(int64_t routes) { return (int)((routes + kChunk - 1) / kChunk); }

}  // namespace

int64_t sorting_workspace_bytes(int tokens, int num_experts, int topk) {
    int64_t routes = (int64_t)tokens * topk;
    if (routes <= kSingleMaxRoutes) return 0;
    return ((int64_t)num_chunks(routes) * num_experts + num_experts) * (int64_t)sizeof(int);
}

void launch_moe_sorting(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                        aiter_tensor_t* sorted_ids, aiter_tensor_t* sorted_w,
                        aiter_tensor_t* sorted_eids, aiter_tensor_t* num_valid,
                        aiter_tensor_t* moe_buf, int E, int unit, const aiter_tensor_t* mask,
                        const aiter_tensor_t* num_local, aiter_tensor_t* workspace,
                        aiter_tensor_t* local_topk_ids, cudaStream_t stream) {
    check_tensor(topk_ids, "topk_ids", AITER_DTYPE_i32, 2);
    check_tensor(topk_weights, "topk_weights", -1, 2);
    B200_CHECK(topk_weights->dtype_ == AITER_DTYPE_fp32, "topk_weights must be FP32 (float32)");
    check_tensor(sorted_ids, "sorted_token_ids", AITER_DTYPE_i32, 1);
    check_tensor(sorted_w, "sorted_weights", AITER_DTYPE_fp32, 1);
    check_tensor(sorted_eids, "sorted_expert_ids", AITER_DTYPE_i32, 1);
    check_tensor(num_valid, "num_valid_ids", AITER_DTYPE_i32, 1);
    const int64_t M = topk_ids->shape[0], topk = topk_ids->shape[1];
    B200_CHECK(topk_weights->shape[0] == M && topk_weights->shape[1] == topk,
               "topk_weights must have the [tokens, topk] shape of topk_ids");
    B200_CHECK(E >= 1 && E <= kMaxExperts, "num_experts must be in [1, ", kMaxExperts, "], got ", E);
    B200_CHECK(unit >= 1, "unit_size must be positive, got ", unit);
    // ids pack the token in 24 bits and the slot in 8 (csrc/include/moe_sorting_opus.h:273-274)
    B200_CHECK(M < (1 << 24), "tokens must be < 2^24, got ", M);
    B200_CHECK(topk >= 1 && topk < 256, "topk must be in [1, 255], got ", topk);
    const int64_t max_padded = M * topk + (int64_t)E * unit - topk;
    B200_CHECK(max_padded < (int64_t)1 << 31, "problem too large");
    const int64_t max_blocks = (max_padded + unit - 1) / unit;
    B200_CHECK((int64_t)sorted_ids->numel_ >= max_padded, "sorted_token_ids needs ", max_padded,
               " elements, has ", sorted_ids->numel_);
    B200_CHECK((int64_t)sorted_w->numel_ >= max_padded, "sorted_weights needs ", max_padded,
               " elements, has ", sorted_w->numel_);
    B200_CHECK((int64_t)sorted_eids->numel_ >= max_blocks, "sorted_expert_ids needs ", max_blocks,
               " elements, has ", sorted_eids->numel_);
    B200_CHECK(num_valid->numel_ >= 2, "num_valid_ids needs 2 elements");
    if (mask) {
        check_tensor(mask, "local_expert_mask", AITER_DTYPE_i32, 1);
        B200_CHECK((int64_t)mask->numel_ == E, "local_expert_mask must have num_experts entries");
    }
    if (num_local) {
        check_tensor(num_local, "num_local_tokens", AITER_DTYPE_i32, -1);
        B200_CHECK(num_local->numel_ >= 1, "num_local_tokens is empty");
    }
    if (local_topk_ids) {
        check_tensor(local_topk_ids, "local_topk_ids", AITER_DTYPE_i32, 2);
        B200_CHECK(local_topk_ids->shape[0] == M && local_topk_ids->shape[1] == topk,
                   "local_topk_ids must have the same [tokens, topk] shape as topk_ids");
    }

    SortArgs a{};
    a.ids = (const int*)topk_ids->ptr;
    a.weights = (const float*)topk_weights->ptr;
    a.mask = mask ? (const int*)mask->ptr : nullptr;
    a.num_local = num_local ? (const int*)num_local->ptr : nullptr;
    a.sorted_ids = (int*)sorted_ids->ptr;
    a.sorted_w = (float*)sorted_w->ptr;
    a.sorted_eids = (int*)sorted_eids->ptr;
    a.num_valid = (int*)num_valid->ptr;
    a.local_topk_ids = local_topk_ids ? (int*)local_topk_ids->ptr : nullptr;
    a.M = (int)M;
    a.topk = (int)topk;
    a.E = E;
    a.unit = unit;
    a.max_padded = (int)max_padded;
    a.max_blocks = (int)max_blocks;

    int zero_ctas = 0;
    if (moe_buf && moe_buf->numel_ > 0) {
        check_tensor(moe_buf, "moe_buf", -1, -1);
        size_t esz = (moe_buf->dtype_ == AITER_DTYPE_fp32 || moe_buf->dtype_ == AITER_DTYPE_i32 ||
                      moe_buf->dtype_ == AITER_DTYPE_u32) ? 4
                   : (moe_buf->dtype_ == AITER_DTYPE_bf16 || moe_buf->dtype_ == AITER_DTYPE_fp16 ||
                      moe_buf->dtype_ == AITER_DTYPE_i16) ? 2
                   : (moe_buf->dtype_ == AITER_DTYPE_i64 || moe_buf->dtype_ == AITER_DTYPE_u64) ? 8 : 1;
        size_t bytes = moe_buf->numel_ * esz;
        B200_CHECK(((uintptr_t)moe_buf->ptr & 15) == 0, "moe_buf must be 16-byte aligned");
        a.zero_buf = (uint4*)moe_buf->ptr;
        a.zero_vec16 = bytes / 16;
        a.zero_tail = (unsigned char*)moe_buf->ptr + a.zero_vec16 * 16;
        a.zero_tail_bytes = (int)(bytes % 16);
        size_t want = (a.zero_vec16 + kThreads * 8 - 1) / (kThreads * 8);
        int cap = 2 * sm_count(topk_ids->device_id);
        zero_ctas = (int)(want < 1 ? 1 : (want > (size_t)cap ? (size_t)cap : want));
    }

    const int64_t routes = M * topk;
    const size_t smem_full = ((size_t)kWarps * E + 2 * (size_t)E + 40) * sizeof(int);
    if (routes <= kSingleMaxRoutes) {
        a.nchunks = 1;
        B200_CUDA(cudaFuncSetAttribute(sort_single_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_full));
        sort_single_kernel<<<1 + zero_ctas, kThreads, smem_full, stream>>>(a);
    } else {
        a.nchunks = num_chunks(routes);
        const int64_t need = sorting_workspace_bytes((int)M, E, (int)topk);
        B200_CHECK(workspace != nullptr && workspace->ptr != nullptr,
                   "workspace of ", need, " bytes is required for this problem size");
        check_tensor(workspace, "workspace", -1, -1);
        B200_CHECK(((uintptr_t)workspace->ptr & 3) == 0, "workspace must be 4-byte aligned");
        size_t ws_esz = (workspace->dtype_ == AITER_DTYPE_u8 || workspace->dtype_ == AITER_DTYPE_i8) ? 1 : 4;
        B200_CHECK((int64_t)(workspace->numel_ * ws_esz) >= need, "workspace needs ", need, " bytes");
        a.ws_cnt = (int*)workspace->ptr;
        a.ws_base = a.ws_cnt + (size_t)a.nchunks * E;
        B200_CUDA(cudaFuncSetAttribute(sort_count_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_full));
        B200_CUDA(cudaFuncSetAttribute(sort_scatter_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_full));
        sort_count_kernel<<<a.nchunks, kThreads, smem_full, stream>>>(a);
        sort_scan_kernel<<<1 + zero_ctas, kThreads, (2 * (size_t)E + 40) * sizeof(int), stream>>>(a);
        sort_scatter_kernel<<<a.nchunks, kThreads, smem_full, stream>>>(a);
    }
    B200_CUDA(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// Sorting without any allocation by anybody.
//
// Some callers have no way to hand over a workspace: a host runtime that reaches this library over
// an FFI and owns no device allocator of its own, a serving loop whose memory pool is frozen after
// start-up, or code that must not trigger the implicit device synchronisation of cudaMalloc/cudaFree
// in the middle of its steady state.  For them the multi-CTA sort keeps its per-chunk counters in a
// fixed array that is part of the loaded module.  Every GPU that loads the library holds these
// kStaticScratchInts * 4 bytes until the process exits.
//
// The name g_sort_scratch is only a host-side handle: the kernels get the real device address from
// cudaGetSymbolAddress, looked up once per device with that device current.
constexpr int kStaticMaxChunks = 64;                       // 64 chunks x 4096 routes = 262144 routes
constexpr int kStaticScratchInts = kStaticMaxChunks * kMaxExperts + kMaxExperts;   // 260 KiB
static __device__ __align__(256) int g_sort_scratch[kStaticScratchInts];

int64_t static_scratch_bytes() { return (int64_t)kStaticScratchInts * (int64_t)sizeof(int); }

// Device address of the scratch array on `dev` (which must be the current device).
static int* static_scratch_ptr(int dev) {
    static int* cached[64] = {nullptr};
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
    void* ptr = nullptr;
    B200_CUDA(cudaGetSymbolAddress(&ptr, g_sort_scratch));
    B200_CHECK(ptr != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    if (dev >= 0 && dev < 64) cached[dev] = (int*)ptr;
    return (int*)ptr;
}

void launch_moe_sorting_noalloc(const aiter_tensor_t* topk_ids, const aiter_tensor_t* topk_weights,
                                aiter_tensor_t* sorted_ids, aiter_tensor_t* sorted_w,
                                aiter_tensor_t* sorted_eids, aiter_tensor_t* num_valid,
                                aiter_tensor_t* moe_buf, int E, int unit, const aiter_tensor_t* mask,
                                const aiter_tensor_t* num_local, aiter_tensor_t* local_topk_ids,
                                cudaStream_t stream) {
    check_tensor(topk_ids, "topk_ids", AITER_DTYPE_i32, 2);
    const int64_t M = topk_ids->shape[0], topk = topk_ids->shape[1];
    B200_CHECK(E >= 1 && E <= kMaxExperts, "num_experts must be in [1, ", kMaxExperts, "], got ", E);
    const int64_t need = sorting_workspace_bytes((int)M, E, (int)topk);
    // stated limit: 262144 routes (tokens*topk); with that and E <= 1024 the scratch always suffices
    B200_CHECK(M * topk <= (int64_t)kStaticMaxChunks * kChunk && need <= static_scratch_bytes(),
               "problem too large for the built-in scratch: ", M * topk, " routes (tokens*topk), the limit is ",
               (int64_t)kStaticMaxChunks * kChunk, " with up to ", kMaxExperts, " experts (", static_scratch_bytes(),
               " bytes held by the library); use b200_moe_sorting_fwd with a caller-provided workspace instead");
    // Nothing in the scratch has to start at zero: the count kernel writes every counter it covers
    // and the scan kernel every base before anything reads them.
    aiter_tensor_t ws{};
    ws.ptr = static_scratch_ptr(topk_ids->device_id);
    ws.numel_ = (size_t)static_scratch_bytes();
    ws.ndim = 1;
    ws.shape[0] = (int64_t)ws.numel_;
    ws.strides[0] = 1;
    ws.dtype_ = AITER_DTYPE_u8;
    ws.device_id = topk_ids->device_id;
    launch_moe_sorting(topk_ids, topk_weights, sorted_ids, sorted_w, sorted_eids, num_valid, moe_buf, E, unit,
                       mask, num_local, need > 0 ? &ws : nullptr, local_topk_ids, stream);
}

}  // namespace b200
