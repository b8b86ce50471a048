// Grouped FP8 block-scaled GEMMs of the fused-MoE layer for sm_100a (tcgen05 + TMEM + TMA).
//
//   stage 1: for every sorted 128-row block (one expert):  [gate|up] = A1 . W1_e^T, then
//            SiLU(gate)*up -> bf16 rounding -> 1x128 FP8 requantisation, written in sorted order
//   stage 2: [128 x 256] = A2 . W2_e^T, times the route weight, added into fp32 acc[token]
//
// Replaces the reference's CK DeviceMoeGemmBlockScale instances
// (csrc/ck_gemm_moe_2stages_codegen/gemm_moe_ck2stages_common_blockscale.cuh:25-169,335-466)
// and follows the arithmetic of its torch oracle (aiter/fused_moe.py:3532-3811).
//
// One persistent CTA per SM walks tiles (block, n-tile) = (t / n_tiles, t % n_tiles), t = blockIdx.x,
// blockIdx.x + gridDim.x, ...; the tile count comes from num_valid_ids on the device (no host sync).
// Per tile and per 128-wide K block:
//   warp 0      TMA-loads two [128 rows x 128 B] weight boxes (gate+up rows, or 256 output rows)
//               into a 128B-swizzled shared-memory stage;
//   warps 4-7   gather the 128 activation rows of the block (cp.async, 16 B chunks, same swizzle);
//               completion is signalled by cp.async.mbarrier.arrive;
//   warp 1      issues 4 tcgen05.mma (M128 N256 K32, e4m3 -> fp32) into one of two 256-column
//               TMEM stages, then commits to free the smem stage and to publish the TMEM stage;
//   warps 8-15  read the TMEM stage (tcgen05.ld) and fold it into fp32 registers with the block
//               scales:  acc += partial * (a_scale[row, kb] * w_scale[e, nblk, kb])  (the scales are read
//               from global memory one K block ahead).
// The scales are fp32 per 128-K block (not UE8M0 per 32), so the hardware block-scaled MMA kinds do
// not apply; the per-K-block promotion runs on the CUDA cores and overlaps the next block's MMAs.
// After the last K block the same warps run the stage's epilogue from registers.
//
// All mbarrier waits are bounded (sm100_ptx.cuh); if one runs out, status[0] is set and the kernel
// winds down: every role leaves its loops, the CTA meets at the tail and frees its TMEM.

#include <cuda_fp8.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;            // sorted rows per tile (== sort unit)
constexpr int BK = 128;            // K elements (bytes) per pipeline step == scale block
constexpr int BN = 256;            // UMMA N: 128 gate + 128 up columns, or 256 output columns
constexpr int kStages = 3;         // shared-memory pipeline depth (4 measured no faster; the space stages stage 2's output)
constexpr int kABytes = BM * BK;   // 16 KB
constexpr int kBBytes = BN * BK;   // 32 KB
constexpr int kThreads = 512;
constexpr int kGatherWarp0 = 4;    // warps 4..7
constexpr int kEpiWarp0 = 8;       // warps 8..15
constexpr int kEpiThreads = 256;
constexpr int kTmemCols = 512;     // 2 stages x 256 fp32 columns
// Registers per thread of each role after setmaxnreg. A CTA's pool is what the launch gave it (registers per thread
// of the compiled kernel x threads); setmaxnreg.inc BLOCKS until the pool covers the request, for ever if the other
// roles never release enough, so the sum is checked at compile time against the launch bound and again at the
// first launch against what the compiler really assigned.
constexpr int kRegsLoad = 24, kRegsGather = 56, kRegsPromo = 216;
constexpr int kRegDemand = 32 * (kGatherWarp0 * kRegsLoad + (kEpiWarp0 - kGatherWarp0) * kRegsGather +
                                 (kThreads / 32 - kEpiWarp0) * kRegsPromo);
static_assert(kRegDemand <= 65536 && kRegDemand <= kThreads * (65536 / kThreads),
              "setmaxnreg: the roles ask for more registers than the CTA is launched with");
constexpr int kTmaSleepNs = 0;         // the single TMA thread polls without back-off
constexpr int kProducerSleepNs = 100;  // back-off of the load roles while no stage is free
#ifndef B200_EPI_SLEEP_NS
#define B200_EPI_SLEEP_NS 40
#endif
constexpr int kEpilogueSleepNs = B200_EPI_SLEEP_NS;   // back-off of the promotion warps while the UMMAs run
constexpr uint32_t kIdesc = ptx::make_idesc_e4m3_f32(BM, BN);

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int kOffA = 0;
constexpr int kOffB = kOffA + kStages * kABytes;
constexpr int kOffBar = kOffB + kStages * kBBytes;          // mbarriers (8 B each)
constexpr int kNumBars = 2 * kStages + 4;
constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr int kOffAbort = kOffTmemSlot + 4;
constexpr int kOffAmax = (kOffAbort + 4 + 15) & ~15;        // float [2 tiles][2 halves][128 rows]
constexpr int kOffRowTab = kOffAmax + 2 * 2 * BM * 4;       // uint32 [2 tiles][128 rows]
constexpr int kStageRowBytes = 272;                            // staged output row: 64 floats + 16 B (bank spread)
constexpr int kOffStage = (kOffRowTab + 2 * BM * 4 + 15) & ~15;   // [8 warps][32 rows][kStageRowBytes] (stage 2)
constexpr int kSmemUsed = kOffStage + 8 * 32 * kStageRowBytes;
constexpr int kSmemBytes = kSmemUsed + 1024;                // slack for the 1024-byte alignment

struct GemmParams {
    const uint8_t* a;        // stage 1: a1 [M,K] by token; stage 2: a2 [P,K] by sorted row
    const float* a_scale;    // [rows, K/128]
    const float* w_scale;    // [E, n_rows/128, K/128]
    const int* sorted_ids;
    const float* sorted_w;
    const int* sorted_eids;
    const int* num_valid;    // {padded total, tokens}
    int M;                   // static token count
    int K, KB;               // K and K/128
    int n_tiles;             // n-tiles this launch covers: stage 1 I/128; stage 2 ceil(columns/256)
    int nt0;                 // first n-tile of this launch (stage 2 column range), else 0
    int acc_ld;              // row pitch of acc in floats (stage 2)
    int n_rows;              // weight rows per expert: 2I (stage 1) or H (stage 2)
    int inter;               // I
    uint8_t* a2;             // stage 1 out [P, I] fp8
    float* a2_scale;         // stage 1 out [P, I/128]
    float* acc;              // stage 2 out [M, H] fp32
    int* status;
    int use_weight;          // multiply this stage's GEMM result by the route weight (sorted_w)
    long long wait_limit;    // SM clocks after which a device-side wait gives up (sets status, the CTA winds down)
    int stall_producer;      // self-test only: the weight producer loads nothing, so every wait downstream runs out
};

// torch: silu(x) = x / (1 + exp(-x)) in fp32, then * up (aiter/fused_moe.py:3676).
// The quotient is formed from an approximate reciprocal and one FMA residual correction (error below
// one fp32 ulp, like the exp it depends on) instead of the ~4x longer IEEE division sequence.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {   // valid for g >= -80
    const float d = 1.0f + expf(-g);
    const float y = ptx::rcp_approx(d);
    const float q = g * y;
    return fmaf(fmaf(-q, d, g), y, q) * u;
}
__device__ __forceinline__ float silu_mul_exact(float g, float u) { return __fdiv_rn(g, 1.0f + expf(-g)) * u; }

// torch: gelu(x) = 0.5 * x * (1 + erf(x / sqrt(2))) (the reference's get_torch_act(Gelu) = F.gelu), then * up
__device__ __forceinline__ float gelu_mul(float g, float u) {
    return 0.5f * g * (1.0f + erff(g * 0.70710678118654752440f)) * u;
}

// act(g) * u for N values. The SiLU fast path is straight-line code, so the N dependency chains (exp,
// reciprocal, two FMAs: ~150 clocks each) interleave; the exact path for exp(-g) near overflow sits behind
// ONE branch per group. With a branch per value every chain is a basic block of its own and the epilogue runs
// at the latency of one chain per value (measured: 9.5k of 11.6k clocks per tile).
template <int ACT, int N>
__device__ __forceinline__ void act_mul_n(const float (&g)[N], const float (&u)[N], float (&h)[N]) {
    if (ACT == 1) {
#pragma unroll
        for (int i = 0; i < N; ++i) h[i] = gelu_mul(g[i], u[i]);
        return;
    }
    float gmin = g[0];
#pragma unroll
    for (int i = 1; i < N; ++i) gmin = fminf(gmin, g[i]);
#pragma unroll
    for (int i = 0; i < N; ++i) h[i] = silu_mul_fast(g[i], u[i]);
    if (gmin < -80.0f) {
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (g[i] < -80.0f) h[i] = silu_mul_exact(g[i], u[i]);
    }
}

// Correctly rounded a / b given rb = RN(1/b): two FMA residual corrections (the first makes the
// quotient faithful, the second then rounds it correctly), valid while nothing over- or underflows.
__device__ __forceinline__ float div_rn_by(float a, float b, float rb) {
    float q = a * rb;
    q = fmaf(fmaf(-q, b, a), rb, q);
    return fmaf(fmaf(-q, b, a), rb, q);
}

// acc[0..7] += v[0..15] * s with packed fp32x2 FMAs (one instruction per column pair)
__device__ __forceinline__ void fold16(float2* acc, const uint32_t* v, float2 s) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
        acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), s, acc[j]);
}

// PT = false: 1x128 activation scales and 128x128 weight scales (QuantType.per_1x128 / per_128x128).
// PT = true : one scale per activation row and one per weight output channel (QuantType.per_Token); the
//             row scale rides on every K step, the channel scales are applied once in the epilogue, and
//             stage 1 writes bf16 (the row-wise requantisation needs the whole row and is a kernel of its own).
// ACT (stage 1 only): 0 = SiLU, 1 = GELU. A compile-time choice: with both bodies in one kernel the 64-fold
//             unrolled epilogue doubles in size and the SiLU path measurably slows down.
template <int STAGE, bool PT, int ACT>
__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = ptx::smem_u32(smem);
    const uint32_t sA = sbase + kOffA, sB = sbase + kOffB;
    const uint32_t bar0 = sbase + kOffBar;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kOffTmemSlot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
    float* amax_x = reinterpret_cast<float*>(smem + kOffAmax);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(full_bar(s), BM + 1);   // 128 gather threads + the TMA thread
            ptx::mbar_init(empty_bar(s), 1);       // one tcgen05.commit
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(tfull_bar(s), 1);                 // one tcgen05.commit
            ptx::mbar_init(tempty_bar(s), kEpiThreads / 32); // one arrive per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_w);
    }
    if (warp == 2) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_valid = p.num_valid[0];
    const int tokens = min(p.num_valid[1], p.M);
    const int total_tiles = (num_valid / BM) * p.n_tiles;

    if (warp < kGatherWarp0) {
        ptx::setmaxnreg_dec<kRegsLoad>();
        if (warp == 0 && lane == 0) {
            // ---------------------------------------------------------------- weight TMA producer
            auto tile_rows = [&](int t, int& r0, int& r1) {
                const int blk = t / p.n_tiles, nt = t - blk * p.n_tiles + p.nt0;
                const int e = p.sorted_eids[blk];
                if (STAGE == 1) {
                    r0 = e * p.n_rows + nt * 128;   // gate rows
                    r1 = r0 + p.inter;              // up rows
                } else {
                    r0 = e * p.n_rows + nt * 256;
                    r1 = (nt * 256 + 128 < p.n_rows) ? r0 + 128 : r0;
                }
            };
            uint32_t it = 0;
            bool ok = !p.stall_producer;   // self-test: issue nothing; the other roles' waits then run out
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                int r0, r1;
                tile_rows(t, r0, r1);
                for (int kb = 0; kb < p.KB; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!(ok = ptx::mbar_wait<kTmaSleepNs>(empty_bar(s), ph ^ 1u, abort_flag, p.wait_limit))) break;
                    ptx::mbar_arrive_expect_tx(full_bar(s), kBBytes);
                    ptx::tma_load_2d(sB + s * kBBytes, &tmap_w, kb * BK, r0, full_bar(s));
                    ptx::tma_load_2d(sB + s * kBBytes + kBBytes / 2, &tmap_w, kb * BK, r1, full_bar(s));
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------------------------------------------------------- UMMA issuer
            // Block scales (PT = false): every K block's partial sums go to the TMEM stage of that step's parity
            // and are promoted in registers. Row/channel scales (PT = true) do not depend on K: the whole K loop
            // accumulates in one TMEM stage, stages alternate per TILE, and the epilogue of a tile overlaps the
            // MMAs of the next.
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++tile_it) {
                for (int kb = 0; kb < p.KB; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    const uint32_t tcount = PT ? tile_it : it;   // what the TMEM stage ring counts
                    const int ts = tcount & 1;
                    const uint32_t tph = (tcount >> 1) & 1u;
                    if (!PT || kb == 0)
                        if (!(ok = ptx::mbar_wait(tempty_bar(ts), tph ^ 1u, abort_flag, p.wait_limit))) break;
                    if (!(ok = ptx::mbar_wait(full_bar(s), ph, abort_flag, p.wait_limit))) break;
                    // the activation rows were written by cp.async (generic proxy); order them
                    // before the tensor core's async-proxy reads
                    ptx::fence_proxy_async();
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::make_kmajor_sw128_desc(sA + s * kABytes);
                    const uint64_t db = ptx::make_kmajor_sw128_desc(sB + s * kBBytes);
                    const uint32_t d = tmem_base + ts * BN;
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)   // 32 bytes of K per UMMA: +2 in 16-byte units
                        ptx::umma_f8(d, da + 2u * k, db + 2u * k, kIdesc, (k > 0 || (PT && kb > 0)) ? 1u : 0u);
                    ptx::umma_commit(empty_bar(s));
                    if (!PT || kb == p.KB - 1) ptx::umma_commit(tfull_bar(ts));
                }
            }
        }
    } else if (warp < kEpiWarp0) {
        // -------------------------------------------------------------------- activation gather
        ptx::setmaxnreg_dec<kRegsGather>();
        const int r = threadIdx.x - kGatherWarp0 * 32;   // row whose scale / row offset this thread owns
        // Copy mapping: 8 consecutive lanes fetch the eight 16-byte chunks of one 128-byte row segment,
        // so a warp-wide cp.async touches 4 whole cache lines (not 32 partial ones). Pass i of a
        // thread covers row gw*32 + i*4 + lane/8.
        const int gw = r >> 5, sub = (r & 31) >> 3;
        const uint32_t chunk = (uint32_t)(r & 7);
        uint32_t* row_tab = reinterpret_cast<uint32_t*>(smem + kOffRowTab);   // [2][128] source rows
        uint32_t it = 0;
        uint32_t tile_par = 0;
        bool ok = true;
        int sid_next = 0;   // sorted id of this thread's row in the next tile, fetched one tile ahead
        if (STAGE == 1 && (int)blockIdx.x < total_tiles)
            sid_next = p.sorted_ids[((int)blockIdx.x / p.n_tiles) * BM + r];
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, tile_par ^= 1u) {
            const int blk = t / p.n_tiles, nt = t - blk * p.n_tiles + p.nt0;
            const int prow = blk * BM + r;
            uint32_t my_row;                 // source row of tile row r, or 0xFFFFFFFF for padding
            if (STAGE == 1) {
                const int tok = sid_next & 0xFFFFFF;
                my_row = tok < tokens ? (uint32_t)tok : 0xFFFFFFFFu;
                if (t + (int)gridDim.x < total_tiles)
                    sid_next = p.sorted_ids[((t + (int)gridDim.x) / p.n_tiles) * BM + r];
            } else {
                my_row = (uint32_t)prow;
            }
            row_tab[tile_par * BM + r] = my_row;
            ptx::named_barrier(2, BM);       // the 128 gather threads; table of the previous tile is
                                             // untouched (other parity), so one barrier per tile suffices
            // source of pass i in 16-byte units from p.a (32 bits cover 64 GB), validity as a bit mask, and the
            // two swizzled destination offsets (even / odd pass): few registers, this role runs with 56
            uint32_t src16[8], vmask = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t sr = row_tab[tile_par * BM + gw * 32 + i * 4 + sub];
                const bool live = sr != 0xFFFFFFFFu;   // pads: zero-filled rows
                vmask |= (live ? 1u : 0u) << i;
                src16[i] = (live ? sr : 0u) * (uint32_t)(p.K >> 4) + chunk;
            }
            const uint32_t row0 = (uint32_t)(gw * 32 + sub);   // row of pass i: row0 + 4 i, so (row & 7) = sub or 4 + sub
            const uint32_t d_even = row0 * BK + ((chunk ^ (uint32_t)sub) << 4);
            const uint32_t d_odd = row0 * BK + ((chunk ^ (uint32_t)(4 + sub)) << 4);
            for (int kb = 0; kb < p.KB; ++kb, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (it / kStages) & 1u;
                if (!(ok = ptx::mbar_wait<kProducerSleepNs>(empty_bar(s), ph ^ 1u, abort_flag, p.wait_limit))) break;
                const uint32_t dst = sA + s * kABytes;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    ptx::cp_async16(dst + ((i & 1) ? d_odd : d_even) + i * 4 * BK, p.a + ((size_t)src16[i] << 4) + (size_t)kb * BK,
                                    ((vmask >> i) & 1u) ? 16u : 0u);
                // the arrival is delivered by the copy engine when this thread's copies have landed,
                // so the thread can go on to the next stage at once (all kStages stay in flight)
                ptx::cp_async_mbar_arrive(full_bar(s));
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();   // nothing of this thread is in flight when the CTA winds down
    } else {
        // -------------------------------------------------------------------- promotion + epilogue
        ptx::setmaxnreg_inc<kRegsPromo>();
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int half = (warp - kEpiWarp0) >> 2;       // which 64 columns of each 128-column group
        const int r = q * 32 + lane;                    // row of the tile == TMEM lane
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t it = 0;
        uint32_t tile_par = 0;
        bool ok = true;
        // row info of the next tile is fetched one tile ahead, so its latency is off the path between
        // two tiles (where the MMA warp can only run two K steps ahead of these warps)
        int tok_next = 0, eid_next = 0;
        float wgt_next = 0.f;
        if ((int)blockIdx.x < total_tiles) {
            const int prow0 = ((int)blockIdx.x / p.n_tiles) * BM + r;
            tok_next = p.sorted_ids[prow0] & 0xFFFFFF;
            eid_next = p.sorted_eids[(int)blockIdx.x / p.n_tiles];
            if (p.use_weight) wgt_next = p.sorted_w[prow0];
        }
        for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, tile_par ^= 1u) {
            const int blk = t / p.n_tiles, nt = t - blk * p.n_tiles + p.nt0;
            const int prow = blk * BM + r;
            const int tok = tok_next, eid = eid_next;
            const bool valid = tok < tokens;
            // the route weight (stage 2, or stage 1 with doweight_stage1) rides on the per-step scales
            const float wgt = p.use_weight ? (valid ? wgt_next : 0.f) : 1.f;
            if (t + (int)gridDim.x < total_tiles) {
                const int prow1 = ((t + (int)gridDim.x) / p.n_tiles) * BM + r;
                tok_next = p.sorted_ids[prow1] & 0xFFFFFF;
                eid_next = p.sorted_eids[(t + (int)gridDim.x) / p.n_tiles];
                if (p.use_weight) wgt_next = p.sorted_w[prow1];
            }
            // a warp whose 32 rows are all padding (decode: most of them) leaves its accumulators at 0
            const bool warp_live = __any_sync(0xffffffffu, valid);

            // acc[j] holds columns (2j, 2j+1) of this thread's first 64 columns for j < 32 and of
            // its second 64 columns (the other 128-column group) for j >= 32
            float2 acc[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) acc[j] = make_float2(0.f, 0.f);

            // Per-step scales come straight from global memory (L1/L2), fetched one K step ahead: a load from
            // shared memory issued after the UMMA's completion sits ~150 clocks (shared memory is saturated by
            // operand reads and fills) on the path to the first FMA.
            // (32-bit element offsets from the parameter pointers: two registers fewer than pointers)
            const uint32_t a_so = (uint32_t)(valid ? (STAGE == 1 ? tok : prow) : 0) * (uint32_t)(PT ? 1 : p.KB);
            uint32_t w_so = 0, w_so1 = 0;
            if (!PT) {
                const int nb0 = (STAGE == 1) ? nt : nt * 2;
                const int nb1 = (STAGE == 1) ? p.inter / 128 + nt : min(nt * 2 + 1, p.n_rows / 128 - 1);
                w_so = (uint32_t)((eid * (p.n_rows / 128) + nb0) * p.KB);
                w_so1 = w_so + (uint32_t)((nb1 - nb0) * p.KB);
            }
            float pf_a = __ldg(p.a_scale + a_so), pf_w0 = PT ? 1.f : __ldg(p.w_scale + w_so), pf_w1 = PT ? 1.f : __ldg(p.w_scale + w_so1);

            // PT: one pass over the finished accumulators per tile (it counts tiles), else one per K block
            for (int kb = PT ? p.KB - 1 : 0; kb < p.KB; ++kb, ++it) {
                const int ts = it & 1;
                const uint32_t tph = (it >> 1) & 1u;
                if (!(ok = ptx::mbar_wait<kEpilogueSleepNs>(tfull_bar(ts), tph, abort_flag, p.wait_limit))) break;
                ptx::tc_fence_after();
                const float sa = pf_a * wgt;   // wgt is exactly 1 when the stage does not weight
                const float s0 = PT ? sa : sa * pf_w0, s1 = PT ? sa : sa * pf_w1;
                if (!PT && kb + 1 < p.KB) {
                    pf_a = __ldg(p.a_scale + a_so + kb + 1);
                    pf_w0 = __ldg(p.w_scale + w_so + kb + 1);
                    pf_w1 = __ldg(p.w_scale + w_so1 + kb + 1);
                }
                const float2 s0v = make_float2(s0, s0), s1v = make_float2(s1, s1);
                const uint32_t ta = lane_addr + ts * BN + half * 64;
                // load + wait, then packed FMAs.  The packed fp32x2 FMAs matter:
                // they need half the issue slots of scalar FMAs, and with scalar FMAs the two promotion
                // warps that share a scheduler with the UMMA-issuing warp starve it (measured: the UMMA
                // rate halves).
                // Eight 16-column chunks (16, not 32: sixteen fewer live registers keep this loop, which sits at
                // the register limit, free of spills - a few spilled values here cost more than 50 %). Sixteen
                // 8-column chunks in two buffers, the next load in flight during the FMAs, measured 3 % slower.
                uint32_t v[16];
                if (warp_live) {
#pragma unroll
                    for (int c = 0; c < 7; ++c) {
                        ptx::tmem_ld_x16_sync(ta + (c >> 2) * 128 + (c & 3) * 16, v);
                        fold16(acc + 8 * c, v, (c < 4) ? s0v : s1v);
                    }
                    ptx::tmem_ld_x16_sync(ta + 128 + 48, v);
                }
                // all reads of this TMEM stage are done: hand it back to the MMA warp
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty_bar(ts));
                if (warp_live) fold16(acc + 56, v, s1v);
            }
            if (!ok) break;

            if (PT) {
                // weight scales per output channel: column j of the first group is weight row
                // e*n_rows + c0 + j, of the second group c1 + j (all lanes read the same addresses)
                const int e = p.sorted_eids[blk];
                const int c0 = (STAGE == 1) ? nt * 128 + half * 64 : nt * 256 + half * 64;
                const int c1 = (STAGE == 1) ? p.inter + c0 : min(c0 + 128, p.n_rows - 64);
                const float4* w0 = reinterpret_cast<const float4*>(p.w_scale + (size_t)e * p.n_rows + c0);
                const float4* w1 = reinterpret_cast<const float4*>(p.w_scale + (size_t)e * p.n_rows + c1);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float4 a = __ldg(w0 + j), b = __ldg(w1 + j);
                    acc[2 * j] = make_float2(acc[2 * j].x * a.x, acc[2 * j].y * a.y);
                    acc[2 * j + 1] = make_float2(acc[2 * j + 1].x * a.z, acc[2 * j + 1].y * a.w);
                    acc[32 + 2 * j] = make_float2(acc[32 + 2 * j].x * b.x, acc[32 + 2 * j].y * b.y);
                    acc[32 + 2 * j + 1] = make_float2(acc[32 + 2 * j + 1].x * b.z, acc[32 + 2 * j + 1].y * b.w);
                }
            }

            if (STAGE == 1 && PT) {
                // SiLU(gate)*up -> bf16, written in sorted-row order; the row-wise quantisation follows
                uint32_t w[32];
#pragma unroll
                for (int j0 = 0; j0 < 32; j0 += 4) {
                    float g[8], u[8], h[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        g[2 * i] = acc[j0 + i].x; g[2 * i + 1] = acc[j0 + i].y;
                        u[2 * i] = acc[32 + j0 + i].x; u[2 * i + 1] = acc[32 + j0 + i].y;
                    }
                    act_mul_n<ACT, 8>(g, u, h);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 hb = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                        w[j0 + i] = *reinterpret_cast<uint32_t*>(&hb);
                    }
                }
                uint4* dst = reinterpret_cast<uint4*>(p.a2 + ((size_t)prow * p.inter + nt * 128 + half * 64) * 2);
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
            } else if (STAGE == 1) {
                // SiLU(gate)*up in fp32 -> bf16 (RNE) -> 1x128 requant, as the oracle does:
                // aiter/fused_moe.py:3668-3681 then aiter/ops/quant.py:64-94 on the bf16 values.
                float amax = 0.f;
#pragma unroll
                for (int j0 = 0; j0 < 32; j0 += 4) {   // acc[j] is overwritten by the two activations it feeds
                    float g[8], u[8], h[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        g[2 * i] = acc[j0 + i].x; g[2 * i + 1] = acc[j0 + i].y;
                        u[2 * i] = acc[32 + j0 + i].x; u[2 * i + 1] = acc[32 + j0 + i].y;
                    }
                    act_mul_n<ACT, 8>(g, u, h);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float h0 = __bfloat162float(__float2bfloat16_rn(h[2 * i]));
                        const float h1 = __bfloat162float(__float2bfloat16_rn(h[2 * i + 1]));
                        acc[j0 + i] = make_float2(h0, h1);
                        amax = fmaxf(amax, fmaxf(fabsf(h0), fabsf(h1)));
                    }
                }
                float* ax = amax_x + tile_par * (2 * BM);
                ax[half * BM + r] = amax;
                ptx::named_barrier(1, kEpiThreads);
                amax = fmaxf(amax, ax[(half ^ 1) * BM + r]);
                float scale = __fdiv_rn(amax, 448.0f);
                if (scale == 0.f) scale = 1.f;
                uint32_t w[16];
                if (scale > 1e-30f) {
                    // x / scale, correctly rounded, from one exact reciprocal per row
                    const float rs = __frcp_rn(scale);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float2 lo = make_float2(div_rn_by(acc[2 * j].x, scale, rs), div_rn_by(acc[2 * j].y, scale, rs));
                        float2 hi = make_float2(div_rn_by(acc[2 * j + 1].x, scale, rs), div_rn_by(acc[2 * j + 1].y, scale, rs));
                        uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
                        uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
                        w[j] = a | (b << 16);
                    }
                } else {   // subnormal-range scale: the reciprocal would overflow
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float2 lo = make_float2(__fdiv_rn(acc[2 * j].x, scale), __fdiv_rn(acc[2 * j].y, scale));
                        float2 hi = make_float2(__fdiv_rn(acc[2 * j + 1].x, scale), __fdiv_rn(acc[2 * j + 1].y, scale));
                        uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
                        uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
                        w[j] = a | (b << 16);
                    }
                }
                uint4* dst = reinterpret_cast<uint4*>(p.a2 + (size_t)prow * p.inter + nt * 128 + half * 64);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                if (half == 0) p.a2_scale[(size_t)prow * (p.inter / 128) + nt] = scale;
            } else {
                // out[token] += weight * row  (aiter/fused_moe.py:3802-3811) as fp32 reductions in L2; the
                // weight is already in the accumulators (it rode on the per-step scales).
                // A thread holds one row. It writes 64 columns (256 contiguous bytes of the output row) to its own
                // shared-memory row and hands them to the copy engine as ONE asynchronous bulk reduce-add, then the
                // other 64 once the engine has read the first out (the buffer holds half a tile).
                // Measured: an SM gets ~20 B/clock of fp32 reductions into L2 whether they are issued as
                // red.global.v4 from registers or as bulk reductions (plain stores: ~35 B/clock), i.e. ~6k clocks
                // per tile that the MMA warp, at most two K steps ahead, waits out; hiding them needs a buffer
                // for the whole 128 KB tile, which neither shared nor tensor memory has room for.
                const uint32_t srow = sbase + kOffStage + (uint32_t)((warp - kEpiWarp0) * 32 + lane) * kStageRowBytes;
                const int n_groups = (nt * 256 + 128 < p.n_rows) ? 2 : 1;
                if (valid) {
                    float* orow = p.acc + (size_t)tok * p.acc_ld + (nt - p.nt0) * 256 + half * 64;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        if (g < n_groups) {
                            ptx::bulk_wait_read_all();   // the copy engine has read this row's previous contents
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                ptx::st_shared_v4(srow + j * 16, acc[g * 32 + 2 * j].x, acc[g * 32 + 2 * j].y,
                                                  acc[g * 32 + 2 * j + 1].x, acc[g * 32 + 2 * j + 1].y);
                            ptx::fence_proxy_async();
                            ptx::bulk_reduce_add_f32(orow + g * 128, srow, 256);
                            ptx::bulk_commit();
                        }
                    }
                }
            }
        }
        ptx::bulk_wait_all();   // nothing of this thread is in flight when the CTA winds down
    }

    // ------------------------------------------------------------------------ tail
    ptx::tc_fence_before();
    __syncthreads();
    const bool gave_up = *abort_flag != 0;
    if (gave_up && threadIdx.x == 0) atomicExch(p.status, 1);
    if (warp == 2) {
        if (gave_up) {
            // give copies / MMAs still in flight a bounded time to land before TMEM is released
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000LL) {
            }
        }
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------- host
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        B200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
        B200_CHECK(sym != nullptr && qres == cudaDriverEntryPointSuccess,
                   "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D view [rows, K] of an fp8 weight tensor [E, n_rows, K]; boxes of 128 rows x 128 bytes, 128B swizzle. Encoding a map
// costs a few microseconds of host time, so the last maps are kept (per thread) and reused while pointer and shape
// repeat, as they do from layer call to layer call.
CUtensorMap make_weight_map(const void* ptr, uint64_t rows, uint64_t K) {
    struct Entry {
        const void* ptr;
        uint64_t rows, K;
        CUtensorMap map;
    };
    constexpr int kEntries = 16;
    static thread_local Entry cache[kEntries];
    static thread_local int next = 0, used = 0;
    for (int i = 0; i < used; ++i)
        if (cache[i].ptr == ptr && cache[i].rows == rows && cache[i].K == K) return cache[i].map;
    CUtensorMap m;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides,
                                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B200_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
    cache[next] = Entry{ptr, rows, K, m};
    next = (next + 1) % kEntries;
    if (used < kEntries) ++used;
    return m;
}

// Process-wide settings of the wait self-test (b200_moe_debug_config): the limit of every device-side wait in SM
// clocks, and whether the weight producer is stalled. Defaults: the built-in limit, no stall.
long long g_wait_limit = ptx::kWaitLimitCycles;
int g_stall_producer = 0;

template <int STAGE, bool PT, int ACT = 0>
void launch_gemm(const CUtensorMap& tmap, const GemmParams& p, int64_t max_tiles, int dev, cudaStream_t stream,
                 int sm_margin = 0) {
    static bool attr_set[64] = {false};
    if (dev >= 64 || !attr_set[dev]) {
        B200_CUDA(cudaFuncSetAttribute(moe_gemm_kernel<STAGE, PT, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes));
        cudaFuncAttributes fa;
        B200_CUDA(cudaFuncGetAttributes(&fa, moe_gemm_kernel<STAGE, PT, ACT>));
        B200_CHECK((int64_t)fa.numRegs * kThreads >= kRegDemand, "GEMM kernel was compiled with ", fa.numRegs,
                   " registers per thread: its roles' setmaxnreg requests (", kRegDemand, " per CTA) could never be met");
        if (dev < 64) attr_set[dev] = true;
    }
    B200_CHECK(sm_margin < sm_count(dev), "sm_margin (", sm_margin, ") must leave at least one of the device's ",
               sm_count(dev), " SMs to the kernel");
    int64_t grid = sm_count(dev) - sm_margin;   // SMs left free for a collective running beside this kernel
    if (max_tiles < grid) grid = max_tiles;
    if (grid < 1) return;
    GemmParams q = p;
    q.wait_limit = g_wait_limit;
    q.stall_producer = g_stall_producer;
    moe_gemm_kernel<STAGE, PT, ACT><<<(unsigned)grid, kThreads, kSmemBytes, stream>>>(tmap, q);
    B200_CUDA(cudaGetLastError());
}

}  // namespace

void set_gemm_debug(long long wait_limit_cycles, int stall_producer) {
    g_wait_limit = wait_limit_cycles > 0 ? wait_limit_cycles : ptx::kWaitLimitCycles;
    g_stall_producer = stall_producer != 0;
}

void launch_moe_stage1(const aiter_tensor_t* a1, const aiter_tensor_t* a1_scale, const aiter_tensor_t* w1,
                       const aiter_tensor_t* w1_scale, const aiter_tensor_t* sorted_ids,
                       const aiter_tensor_t* sorted_eids, const aiter_tensor_t* num_valid, aiter_tensor_t* a2,
                       aiter_tensor_t* a2_scale, aiter_tensor_t* status, int quant_type,
                       const aiter_tensor_t* sorted_w, int activation, cudaStream_t stream) {
    B200_CHECK(activation == 0 || activation == 1, "activation must be Silu (0) or Gelu (1), got ", activation);
    if (sorted_w) {
        check_tensor(sorted_w, "sorted_weights", AITER_DTYPE_fp32, 1);
        B200_CHECK(sorted_w->numel_ >= sorted_ids->numel_, "sorted_weights must cover sorted_token_ids");
    }
    // quant_type: QuantType of the reference (csrc/include/aiter_enum.h:16-26): 4/5 = block scale, 2 = per_Token
    B200_CHECK(quant_type == 4 || quant_type == 5 || quant_type == 2,
               "quant_type must be per_1x128 (4), per_128x128 (5) or per_Token (2), got ", quant_type);
    const bool pt = quant_type == 2;
    check_tensor(a1, "a1", AITER_DTYPE_fp8, 2);
    check_tensor(a1_scale, "a1_scale", AITER_DTYPE_fp32, -1);
    check_tensor(w1, "w1", AITER_DTYPE_fp8, 3);
    check_tensor(w1_scale, "w1_scale", AITER_DTYPE_fp32, -1);
    check_tensor(sorted_ids, "sorted_token_ids", AITER_DTYPE_i32, 1);
    check_tensor(sorted_eids, "sorted_expert_ids", AITER_DTYPE_i32, 1);
    check_tensor(num_valid, "num_valid_ids", AITER_DTYPE_i32, 1);
    check_tensor(a2, "a2", pt ? AITER_DTYPE_bf16 : AITER_DTYPE_fp8, 2);
    if (!pt) check_tensor(a2_scale, "a2_scale", AITER_DTYPE_fp32, -1);
    check_tensor(status, "status", AITER_DTYPE_i32, -1);
    const int64_t M = a1->shape[0], H = a1->shape[1];
    const int64_t E = w1->shape[0], N2 = w1->shape[1];
    B200_CHECK(w1->shape[2] == H, "w1 must be [E, 2*inter_dim, model_dim]: K ", w1->shape[2], " != ", H);
    B200_CHECK(N2 % 256 == 0, "2*inter_dim must be a multiple of 256 (inter_dim % 128 == 0), got ", N2);
    B200_CHECK(H % 128 == 0, "model_dim must be a multiple of 128, got ", H);
    const int64_t I = N2 / 2;
    if (pt) {
        B200_CHECK((int64_t)a1_scale->numel_ == M, "a1_scale must have one element per token for per_Token");
        B200_CHECK((int64_t)w1_scale->numel_ == E * N2, "w1_scale must have E*2*inter_dim elements for per_Token");
    } else {
        B200_CHECK((int64_t)a1_scale->numel_ == M * (H / 128), "a1_scale must have M*model_dim/128 elements");
        B200_CHECK((int64_t)w1_scale->numel_ == E * (N2 / 128) * (H / 128),
                   "w1_scale must have E*(2*inter_dim/128)*(model_dim/128) elements");
    }
    const int64_t P = a2->shape[0];
    B200_CHECK(a2->shape[1] == I, "a2 must be [P, inter_dim]");
    B200_CHECK((int64_t)sorted_ids->numel_ >= 1 && P >= (int64_t)sorted_ids->numel_,
               "a2 must have at least as many rows as sorted_token_ids (", sorted_ids->numel_, "), has ", P);
    if (!pt) B200_CHECK((int64_t)a2_scale->numel_ >= P * (I / 128), "a2_scale must have P*inter_dim/128 elements");
    B200_CHECK(num_valid->numel_ >= 2 && status->numel_ >= 1, "num_valid_ids needs 2 and status 1 element");
    B200_CHECK((int64_t)sorted_eids->numel_ * BM >= (int64_t)sorted_ids->numel_ - (BM - 1),
               "sorted_expert_ids must hold one entry per 128 sorted rows (was the sort run with unit_size 128?)");
    B200_CHECK(E * N2 < ((int64_t)1 << 31) && M < (1 << 24), "problem too large");
    B200_CHECK(((uintptr_t)a1->ptr & 15) == 0 && ((uintptr_t)w1->ptr & 15) == 0 && ((uintptr_t)a2->ptr & 15) == 0 &&
                   ((uintptr_t)w1_scale->ptr & 15) == 0,
               "a1, w1, w1_scale and a2 must be 16-byte aligned");

    GemmParams p{};
    p.a = (const uint8_t*)a1->ptr;
    p.a_scale = (const float*)a1_scale->ptr;
    p.w_scale = (const float*)w1_scale->ptr;
    p.sorted_ids = (const int*)sorted_ids->ptr;
    p.sorted_eids = (const int*)sorted_eids->ptr;
    p.num_valid = (const int*)num_valid->ptr;
    p.M = (int)M;
    p.K = (int)H;
    p.KB = (int)(H / 128);
    p.n_tiles = (int)(I / 128);
    p.n_rows = (int)N2;
    p.inter = (int)I;
    p.a2 = (uint8_t*)a2->ptr;
    p.a2_scale = pt ? nullptr : (float*)a2_scale->ptr;
    p.status = (int*)status->ptr;
    p.sorted_w = sorted_w ? (const float*)sorted_w->ptr : nullptr;
    p.use_weight = sorted_w != nullptr;   // doweight_stage1 (aiter/fused_moe.py:3651-3652)
    CUtensorMap tmap = make_weight_map(w1->ptr, (uint64_t)(E * N2), (uint64_t)H);
    const int64_t max_tiles = ((int64_t)sorted_ids->numel_ / BM) * p.n_tiles;
    if (pt && activation == 1) launch_gemm<1, true, 1>(tmap, p, max_tiles, a1->device_id, stream);
    else if (pt) launch_gemm<1, true, 0>(tmap, p, max_tiles, a1->device_id, stream);
    else if (activation == 1) launch_gemm<1, false, 1>(tmap, p, max_tiles, a1->device_id, stream);
    else launch_gemm<1, false, 0>(tmap, p, max_tiles, a1->device_id, stream);
}

void launch_moe_stage2(const aiter_tensor_t* a2, const aiter_tensor_t* a2_scale, const aiter_tensor_t* w2,
                       const aiter_tensor_t* w2_scale, const aiter_tensor_t* sorted_ids,
                       const aiter_tensor_t* sorted_w, const aiter_tensor_t* sorted_eids,
                       const aiter_tensor_t* num_valid, aiter_tensor_t* acc, aiter_tensor_t* status,
                       int col_begin, int col_end, int sm_margin, int quant_type, int doweight, cudaStream_t stream) {
    B200_CHECK(quant_type == 4 || quant_type == 5 || quant_type == 2,
               "quant_type must be per_1x128 (4), per_128x128 (5) or per_Token (2), got ", quant_type);
    const bool pt = quant_type == 2;
    check_tensor(a2, "a2", AITER_DTYPE_fp8, 2);
    check_tensor(a2_scale, "a2_scale", AITER_DTYPE_fp32, -1);
    check_tensor(w2, "w2", AITER_DTYPE_fp8, 3);
    check_tensor(w2_scale, "w2_scale", AITER_DTYPE_fp32, -1);
    check_tensor(sorted_ids, "sorted_token_ids", AITER_DTYPE_i32, 1);
    check_tensor(sorted_w, "sorted_weights", AITER_DTYPE_fp32, 1);
    check_tensor(sorted_eids, "sorted_expert_ids", AITER_DTYPE_i32, 1);
    check_tensor(num_valid, "num_valid_ids", AITER_DTYPE_i32, 1);
    check_tensor(acc, "acc", AITER_DTYPE_fp32, 2);
    check_tensor(status, "status", AITER_DTYPE_i32, -1);
    const int64_t P = a2->shape[0], I = a2->shape[1];
    const int64_t E = w2->shape[0], H = w2->shape[1];
    const int64_t M = acc->shape[0];
    B200_CHECK(w2->shape[2] == I, "w2 must be [E, model_dim, inter_dim]: K ", w2->shape[2], " != ", I);
    if (col_end <= 0) col_end = (int)H;
    B200_CHECK(col_begin >= 0 && col_begin < col_end && col_end <= H && col_begin % 256 == 0 &&
                   (col_end % 256 == 0 || col_end == H),
               "column range [", col_begin, ", ", col_end, ") must lie in [0, model_dim] on 256-column boundaries");
    // acc is either the range's own block [M, col_end - col_begin] or the whole [M, model_dim] buffer, of which
    // this launch then fills columns [col_begin, col_end)
    const bool full_width = acc->shape[1] == H;
    B200_CHECK(full_width || acc->shape[1] == col_end - col_begin, "acc must be [M, col_end - col_begin] or [M, model_dim]");
    B200_CHECK(((uintptr_t)acc->ptr & 15) == 0, "acc must be 16-byte aligned (bulk reductions)");
    B200_CHECK(sm_margin >= 0, "sm_margin must not be negative");
    B200_CHECK(I % 128 == 0 && H % 128 == 0, "inter_dim and model_dim must be multiples of 128");
    if (pt) {
        B200_CHECK((int64_t)a2_scale->numel_ >= P, "a2_scale must have one element per sorted row for per_Token");
        B200_CHECK((int64_t)w2_scale->numel_ == E * H, "w2_scale must have E*model_dim elements for per_Token");
        B200_CHECK(((uintptr_t)w2_scale->ptr & 15) == 0, "w2_scale must be 16-byte aligned");
    } else {
        B200_CHECK((int64_t)a2_scale->numel_ >= P * (I / 128), "a2_scale must have P*inter_dim/128 elements");
        B200_CHECK((int64_t)w2_scale->numel_ == E * (H / 128) * (I / 128),
                   "w2_scale must have E*(model_dim/128)*(inter_dim/128) elements");
    }
    B200_CHECK(P >= (int64_t)sorted_ids->numel_ && sorted_w->numel_ >= sorted_ids->numel_,
               "a2 and sorted_weights must cover sorted_token_ids");
    B200_CHECK(num_valid->numel_ >= 2 && status->numel_ >= 1, "num_valid_ids needs 2 and status 1 element");
    B200_CHECK((int64_t)sorted_eids->numel_ * BM >= (int64_t)sorted_ids->numel_ - (BM - 1),
               "sorted_expert_ids must hold one entry per 128 sorted rows (was the sort run with unit_size 128?)");
    B200_CHECK(E * H < ((int64_t)1 << 31) && M < (1 << 24), "problem too large");
    B200_CHECK(((uintptr_t)a2->ptr & 15) == 0 && ((uintptr_t)w2->ptr & 15) == 0 && ((uintptr_t)acc->ptr & 15) == 0,
               "a2, w2 and acc must be 16-byte aligned");

    GemmParams p{};
    p.a = (const uint8_t*)a2->ptr;
    p.a_scale = (const float*)a2_scale->ptr;
    p.w_scale = (const float*)w2_scale->ptr;
    p.sorted_ids = (const int*)sorted_ids->ptr;
    p.sorted_w = (const float*)sorted_w->ptr;
    p.sorted_eids = (const int*)sorted_eids->ptr;
    p.num_valid = (const int*)num_valid->ptr;
    p.M = (int)M;
    p.K = (int)I;
    p.KB = (int)(I / 128);
    p.n_tiles = (col_end - col_begin + 255) / 256;
    p.nt0 = col_begin / 256;
    p.acc_ld = full_width ? (int)H : col_end - col_begin;
    p.n_rows = (int)H;
    p.inter = (int)I;
    p.acc = (float*)acc->ptr + (full_width ? col_begin : 0);
    p.status = (int*)status->ptr;
    p.use_weight = doweight != 0;
    CUtensorMap tmap = make_weight_map(w2->ptr, (uint64_t)(E * H), (uint64_t)I);
    const int64_t max_tiles = ((int64_t)sorted_ids->numel_ / BM) * p.n_tiles;
    if (pt) launch_gemm<2, true>(tmap, p, max_tiles, a2->device_id, stream, sm_margin);
    else launch_gemm<2, false>(tmap, p, max_tiles, a2->device_id, stream, sm_margin);
}

}  // namespace b200
