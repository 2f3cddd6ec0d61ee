// Plain and grouped GEMM on the tcgen05 core (see gemm_sm100.cuh): bf16 inputs, or e4m3 inputs
// with 1x128 (activations) and 128x128 (weights) fp32 block scales applied in the epilogue warps.
// The grouped form consumes the expanded (expert-major) output of the dispatch directly:
// `group_end` is the device-resident prefix array of the dispatch handle, so no host
// synchronisation sits between dispatch and the expert GEMM.
//
// The reference library contains no GEMM; this is the compute half of the fused MoE layer and of
// the all-gather -> GEMM / GEMM -> reduce-scatter operators (tp_fused.cu).
#include <cstdlib>

#include "gemm_api.hpp"
#include "gemm_sm100.cuh"

namespace ep {
namespace gemm {

namespace {

struct Tile {
    int g, m0, m_end, n0;
    int kb0, kb1;       // k-blocks [kb0, kb1) of this tile (all of K unless the problem is grouped along K)
};

// Walks the tiles of a (grouped) problem in a fixed order: group, then bands of kBandM m-blocks, inside a band
// n-block then m-block.
struct Scheduler {
    static constexpr int kBandM = 8;
    const GemmParams& p;
    int tiles_n, BN, BM, BK;
    int g = 0, base = 0, start = 0, end = 0;
    __device__ Scheduler(const GemmParams& p_, int bn, int bm = gemm::BM, int bk = 64) : p(p_), tiles_n(p_.N / bn), BN(bn), BM(bm), BK(bk) {
        end = (p.group_end != nullptr && !p.k_grouped) ? p.group_end[0] : p.M;
    }
    __device__ bool get(int t, Tile& out) {
        if (p.k_grouped) {
            // groups along K: every group is a full M x N problem over its own range of k (the rows of one expert)
            const int tiles_m = ceil_div(p.M, BM);
            const int tiles = tiles_m * tiles_n;
            if (t >= p.num_groups * tiles) return false;
            const int gk = t / tiles, local = t % tiles;
            const int band = local / (kBandM * tiles_n), rem = local % (kBandM * tiles_n);
            const int band_m = min(kBandM, tiles_m - band * kBandM);
            out.g = gk;
            out.m0 = (band * kBandM + rem % band_m) * BM;
            out.m_end = p.M;
            out.n0 = (rem / band_m) * BN;
            const int k_start = gk == 0 ? 0 : align_up(p.group_end[gk - 1], p.group_alignment);
            const int k_end = max(p.group_end[gk], k_start);
            out.kb0 = k_start / BK;
            out.kb1 = ceil_div(k_end, BK);
            return true;
        }
        out.kb0 = 0;
        out.kb1 = p.K / BK;
        while (g < p.num_groups) {
            const int rows = max(end - start, 0);
            const int tiles_m = ceil_div(rows, BM);
            const int tiles = tiles_m * tiles_n;
            if (t < base + tiles) {
                const int local = t - base;
                // m-blocks run fastest, in bands of kBandM m-blocks: the tiles that are in flight at the same time
                // then share few A row-blocks AND few B row-blocks, which keeps both resident in L2
                const int band = local / (kBandM * tiles_n), rem = local % (kBandM * tiles_n);
                const int band_m = min(kBandM, tiles_m - band * kBandM);
                out.g = g;
                out.m0 = start + (band * kBandM + rem % band_m) * BM;
                out.m_end = end;
                out.n0 = (rem / band_m) * BN;
                return true;
            }
            base += tiles;
            ++g;
            if (g < p.num_groups) {
                start = align_up(end, p.group_alignment);
                end = p.group_end[g];
            }
        }
        return false;
    }
};

template <int BN, bool kFp8>
struct Cfg {
    static constexpr int kEpiWarps = kFp8 ? 16 : 4;     // FP8: 4 lane quarters x 4 column quarters, so that many passes overlap
    static constexpr int kThreads = (2 + kEpiWarps) * 32;
    static constexpr int BK = kFp8 ? 128 : 64;          // one 128-byte swizzle span per row
    static constexpr int UMMA_K = kFp8 ? 32 : 16;
    static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
    static constexpr int kStages = (192 * 1024) / STAGE;
    // accumulators in tensor memory: two tiles for bf16; with FP8 every k-block is an accumulator pass and the
    // epilogue is the slower side, so four passes may be in flight
    static constexpr int kAccStages = kFp8 ? 4 : 2;
    static constexpr int kBarBytes = (2 * kStages + 2 * kAccStages) * 8 + 16;
    static constexpr int kSmem = kStages * STAGE + kBarBytes + 1024;   // + slack to align the ring to 1024 bytes
    static constexpr int kTmemCols = kAccStages * BN;
};

template <int BN, bool kFp8>
__global__ void __launch_bounds__(Cfg<BN, kFp8>::kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using C = Cfg<BN, kFp8>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kStages * C::STAGE);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;
    uint64_t* tmem_empty = tmem_full + C::kAccStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + C::kAccStages);

    const int warp = warp_id(), lane = lane_id();
    const int num_kb = p.K / C::BK;
    PipeCtx pc{p.error, globaltimer_ns() + p.timeout_ns};

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < C::kAccStages; ++a) {
            mbar_init(tmem_full + a, 1);
            // bf16: every epilogue thread arrives once per tile; FP8: one arrival per warp and k-block (an accumulator
            // pass per k-block makes per-thread arrivals the bottleneck)
            mbar_init(tmem_empty + a, kFp8 ? C::kEpiWarps : C::kEpiWarps * 32);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            Scheduler sched(p, BN, BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
                const int b_row = (p.k_grouped ? 0 : t.g * p.N) + t.n0;
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    mbar_arrive_expect_tx(full + s, C::STAGE);
                    tma_load_2d(sa, &map_a, kb * C::BK, t.m0, full + s);
                    tma_load_2d(sa + C::A_BYTES, &map_b, kb * C::BK, b_row, full + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            Scheduler sched(p, BN, BM, C::BK);
            Tile t;
            constexpr uint32_t idesc = make_idesc<kFp8>(BM, BN);
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
                if constexpr (!kFp8) {
                    if (!(ok = pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1))) break;
                    tc_fence_after();
                }
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if constexpr (kFp8) {
                        if (!(ok = pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1))) break;
                    }
                    if (!(ok = pipe_wait(pc, full + s, ph))) break;
                    tc_fence_after();
                    const uint8_t* sa = smem + s * C::STAGE;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::A_BYTES);
                    const uint32_t d_addr = tmem_base + acc * BN;
#pragma unroll
                    for (int k = 0; k < C::BK / C::UMMA_K; ++k) {
                        const uint32_t accumulate = kFp8 ? (k != 0) : (kb != t.kb0 || k != 0);
                        umma<kFp8>(d_addr, da + 2 * k, db + 2 * k, idesc, accumulate);
                    }
                    umma_commit(empty + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                    if constexpr (kFp8) {
                        umma_commit(tmem_full + acc);
                        if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
                    }
                }
                if constexpr (!kFp8) {
                    if (!ok) break;
                    if (t.kb1 > t.kb0) umma_commit(tmem_full + acc);
                    else mbar_arrive(tmem_full + acc);        // an empty k range: nothing was issued, the epilogue writes zeros
                    if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;                  // the TMEM lanes this warp may read: [32 * quarter, +32)
        const int part = (warp - 2) / 4;               // fp8: which quarter of the columns
        constexpr int kCols = kFp8 ? BN / 4 : BN;      // columns per thread
        Scheduler sched(p, BN, BM, C::BK);
        Tile t;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
            const int row = t.m0 + quarter * 32 + lane;
            const bool row_ok = row < t.m_end && row < p.M;
            const bool zero_row = !row_ok && p.zero_gap && row < p.M;   // alignment gap of the expanded layout
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            __nv_bfloat16* c_row = p.C + (p.k_grouped ? static_cast<int64_t>(t.g) * p.c_group_stride : 0) +
                                   static_cast<int64_t>(row) * p.ldc + t.n0 + part * kCols;
            if constexpr (!kFp8) {
                if (!(ok = pipe_wait(pc, tmem_full + acc, acc_ph))) break;
                tc_fence_after();
                const bool empty_k = t.kb1 <= t.kb0;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(lane_addr + acc * BN + c * 32, r);
                    tmem_ld_wait();
                    if (empty_k) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = 0u;
                    }
                    if (row_ok) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            int4 out;
                            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                            *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = out;
                        }
                    } else if (zero_row) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = make_int4(0, 0, 0, 0);
                    }
                }
                tc_fence_before();
                mbar_arrive(tmem_empty + acc);
                if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
            } else {
                float sum[kCols];
#pragma unroll
                for (int i = 0; i < kCols; ++i) sum[i] = 0.f;
                const int kblocks_b = p.K / 128;
                const float* sfb = p.sfb + (static_cast<int64_t>(t.g) * (p.N / 128) + t.n0 / 128) * kblocks_b;
                const float* sfa = p.sfa + static_cast<int64_t>(row_ok ? row : 0) * p.sfa_row_stride;
                float next_scale = sfa[0] * sfb[0];
                for (int kb = 0; kb < num_kb; ++kb) {
                    const float scale = next_scale;
                    if (kb + 1 < num_kb) next_scale = sfa[static_cast<int64_t>(kb + 1) * p.sfa_k_stride] * sfb[kb + 1];
                    if (!(ok = pipe_wait(pc, tmem_full + acc, acc_ph))) break;
                    tc_fence_after();
                    static_assert(kCols == 32, "the FP8 epilogue is written for 32 columns per thread");
                    uint32_t r0[32];
                    tmem_ld_32x32(lane_addr + acc * BN + part * kCols, r0);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_empty + acc);      // the values are in registers: the accumulator can be reused
                    if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
#pragma unroll
                    for (int i = 0; i < 32; ++i) sum[i] = fmaf(scale, __uint_as_float(r0[i]), sum[i]);
                }
                if (ok && zero_row) {
#pragma unroll
                    for (int v = 0; v < kCols / 8; ++v) *reinterpret_cast<int4*>(c_row + v * 8) = make_int4(0, 0, 0, 0);
                }
                if (ok && row_ok) {
#pragma unroll
                    for (int v = 0; v < kCols / 8; ++v) {
                        int4 out;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(sum[v * 8 + 2 * i], sum[v * 8 + 2 * i + 1]);
                        *reinterpret_cast<int4*>(c_row + v * 8) = out;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ==================================================================== CTA-pair kernel (bf16, 256 x 256 tiles)
// A cluster of two CTAs owns a 256 x 256 tile: CTA r loads rows [128 r, 128 r + 128) of the A tile and of the B tile
// (32 KB per stage instead of 48 KB for a lone CTA, so six stages fit and a third less shared-memory fill traffic
// per flop), the leader's MMA warp issues tcgen05.mma.cta_group::2 (M = 256), each CTA's epilogue warps drain the
// 128 accumulator rows in their own tensor memory. Barriers: `full` lives in the leader and counts the bytes of both
// CTAs; `empty` and `tmem_full` are signalled in both CTAs by one multicast commit; the leader's `tmem_empty`
// collects the epilogue threads of both CTAs.
struct PairCfg {
    static constexpr int BN = 256, BK = 64, UMMA_K = 16;
    static constexpr int A_BYTES = BM * 128, B_BYTES = (BN / 2) * 128, STAGE = A_BYTES + B_BYTES;
    static constexpr int kStages = 6;
    static constexpr int kAccStages = 2;
    static constexpr int kEpiWarps = 4;
    static constexpr int kThreads = (2 + kEpiWarps) * 32;
    static constexpr int kBarBytes = (2 * kStages + 2 * kAccStages) * 8 + 16;
    static constexpr int kSmem = kStages * STAGE + kBarBytes + 1024;
    static constexpr int kTmemCols = kAccStages * BN;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using C = PairCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kStages * C::STAGE);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;
    uint64_t* tmem_empty = tmem_full + C::kAccStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + C::kAccStages);

    const int warp = warp_id(), lane = lane_id();
    const uint32_t cta = cluster_ctarank();
    const bool leader = cta == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = p.K / C::BK;
    PipeCtx pc{p.error, globaltimer_ns() + p.timeout_ns};

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < C::kAccStages; ++a) {
            mbar_init(tmem_full + a, 1);
            mbar_init(tmem_empty + a, 2 * C::kEpiWarps * 32);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();          // barriers of both CTAs are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                const int b_row = (p.k_grouped ? 0 : t.g * p.N) + t.n0 + static_cast<int>(cta) * (C::BN / 2);
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    if (leader) mbar_arrive_expect_tx(full + s, 2 * C::STAGE);
                    const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                    tma_load_2d_pair(sa, &map_a, kb * C::BK, t.m0 + static_cast<int>(cta) * BM, bar);
                    tma_load_2d_pair(sa + C::A_BYTES, &map_b, kb * C::BK, b_row, bar);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            constexpr uint32_t idesc = make_idesc<false>(2 * BM, C::BN);
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                if (!(ok = pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1))) break;
                tc_fence_after();
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, full + s, ph))) break;
                    tc_fence_after();
                    const uint8_t* sa = smem + s * C::STAGE;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::A_BYTES);
                    const uint32_t d_addr = tmem_base + acc * C::BN;
#pragma unroll
                    for (int k = 0; k < C::BK / C::UMMA_K; ++k) umma_pair_bf16(d_addr, da + 2 * k, db + 2 * k, idesc, kb != t.kb0 || k != 0);
                    umma_commit_pair(empty + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                if (t.kb1 > t.kb0) {
                    umma_commit_pair(tmem_full + acc);
                } else {                                     // an empty k range: nothing was issued, the epilogues write zeros
                    mbar_arrive_cluster(map_to_cta(smem_u32(tmem_full + acc), 0));
                    mbar_arrive_cluster(map_to_cta(smem_u32(tmem_full + acc), 1));
                }
                if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (both CTAs, own 128 rows)
        const int quarter = warp & 3;
        Scheduler sched(p, C::BN, 2 * BM, C::BK);
        Tile t;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
            const int row = t.m0 + static_cast<int>(cta) * BM + quarter * 32 + lane;
            const bool row_ok = row < t.m_end && row < p.M;
            const bool zero_row = !row_ok && p.zero_gap && row < p.M && row < align_up(t.m_end, p.group_alignment);
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            __nv_bfloat16* c_row = p.C + (p.k_grouped ? static_cast<int64_t>(t.g) * p.c_group_stride : 0) + static_cast<int64_t>(row) * p.ldc + t.n0;
            if (!(ok = pipe_wait(pc, tmem_full + acc, acc_ph))) break;
            tc_fence_after();
            const bool empty_k = t.kb1 <= t.kb0;
#pragma unroll 1
            for (int c = 0; c < C::BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + acc * C::BN + c * 32, r);
                tmem_ld_wait();
                if (empty_k) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        int4 out;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                        *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = out;
                    }
                } else if (zero_row) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = make_int4(0, 0, 0, 0);
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
            if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
        }
    }

    tc_fence_before();
    cluster_sync_all();          // nobody frees tensor memory, or leaves, while the peer may still signal or read
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

// ==================================================================== CTA-pair kernel, e4m3 with software block scaling (256 x 256 tiles)
// Same division of labour as gemm_pair_kernel; a stage holds a 128-wide k-block (128 bytes per row), and every
// k-block is an accumulator pass of its own (two passes fit into the 512 columns of tensor memory): the leader
// commits the pass, the sixteen epilogue warps of each CTA -- four lane quarters x four column quarters of 64 --
// drain it sixteen columns at a time and add it, times the product of the 1x128 scale of the row and the 128x128
// scale of the weight block, to fp32 sums in registers. Per flop a pair loads a third less than two lone CTAs with
// 128 x 128 tiles would, which is what the FP8 rate needs: the main loop is bound by the fill of shared memory.
struct PairFp8Cfg {
    static constexpr int BN = 256, BK = 128, UMMA_K = 32;
    static constexpr int A_BYTES = BM * 128, B_BYTES = (BN / 2) * 128, STAGE = A_BYTES + B_BYTES;
    static constexpr int kStages = 6;
    static constexpr int kAccStages = 2;
    static constexpr int kEpiWarps = 16;
    static constexpr int kThreads = (2 + kEpiWarps) * 32;
    static constexpr int kBarBytes = (2 * kStages + 2 * kAccStages) * 8 + 16;
    static constexpr int kSmem = kStages * STAGE + kBarBytes + 1024;
    static constexpr int kTmemCols = kAccStages * BN;
    static constexpr int kColsPerThread = BN / 4;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairFp8Cfg::kThreads, 1)
gemm_pair_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using C = PairFp8Cfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kStages * C::STAGE);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;
    uint64_t* tmem_empty = tmem_full + C::kAccStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + C::kAccStages);

    const int warp = warp_id(), lane = lane_id();
    const uint32_t cta = cluster_ctarank();
    const bool leader = cta == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = p.K / C::BK;
    PipeCtx pc{p.error, globaltimer_ns() + p.timeout_ns};

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < C::kAccStages; ++a) {
            mbar_init(tmem_full + a, 1);
            mbar_init(tmem_empty + a, 2 * C::kEpiWarps);      // one arrival per epilogue warp of either CTA and k-block
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    if (leader) mbar_arrive_expect_tx(full + s, 2 * C::STAGE);
                    const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                    tma_load_2d_pair(sa, &map_a, kb * C::BK, t.m0 + static_cast<int>(cta) * BM, bar);
                    tma_load_2d_pair(sa + C::A_BYTES, &map_b, kb * C::BK, t.g * p.N + t.n0 + static_cast<int>(cta) * (C::BN / 2), bar);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only): one accumulator pass per k-block
        if (leader && lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            constexpr uint32_t idesc = make_idesc<true>(2 * BM, C::BN);
            int s = 0, acc = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1))) break;
                    if (!(ok = pipe_wait(pc, full + s, ph))) break;
                    tc_fence_after();
                    const uint8_t* sa = smem + s * C::STAGE;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::A_BYTES);
                    const uint32_t d_addr = tmem_base + acc * C::BN;
#pragma unroll
                    for (int k = 0; k < C::BK / C::UMMA_K; ++k) umma_pair_fp8(d_addr, da + 2 * k, db + 2 * k, idesc, k != 0);
                    umma_commit_pair(empty + s);
                    umma_commit_pair(tmem_full + acc);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                    if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (both CTAs, own 128 rows)
        const int quarter = warp & 3;                  // the TMEM lanes this warp may read: [32 * quarter, +32)
        const int part = (warp - 2) / 4;               // which quarter of the 256 columns
        constexpr int kCols = C::kColsPerThread;
        Scheduler sched(p, C::BN, 2 * BM, C::BK);
        Tile t;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        const int kblocks_b = p.K / 128;
        for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
            const int row = t.m0 + static_cast<int>(cta) * BM + quarter * 32 + lane;
            const bool row_ok = row < t.m_end && row < p.M;
            const bool zero_row = !row_ok && p.zero_gap && row < p.M && row < align_up(t.m_end, p.group_alignment);
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            __nv_bfloat16* c_row = p.C + static_cast<int64_t>(row) * p.ldc + t.n0 + part * kCols;
            float sum[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) sum[i] = 0.f;
            const float* sfb = p.sfb + (static_cast<int64_t>(t.g) * (p.N / 128) + (t.n0 + part * kCols) / 128) * kblocks_b;
            const float* sfa = p.sfa + static_cast<int64_t>(row_ok ? row : 0) * p.sfa_row_stride;
            float next_scale = sfa[0] * sfb[0];
            for (int kb = 0; kb < num_kb; ++kb) {
                const float scale = next_scale;
                if (kb + 1 < num_kb) next_scale = sfa[static_cast<int64_t>(kb + 1) * p.sfa_k_stride] * sfb[kb + 1];
                if (!(ok = pipe_wait(pc, tmem_full + acc, acc_ph))) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < kCols / 16; ++c) {
                    uint32_t r[16];
                    tmem_ld_32x16(lane_addr + acc * C::BN + part * kCols + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) sum[c * 16 + i] = fmaf(scale, __uint_as_float(r[i]), sum[c * 16 + i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
                if (++acc == C::kAccStages) { acc = 0; acc_ph ^= 1; }
            }
            if (ok && zero_row) {
#pragma unroll
                for (int v = 0; v < kCols / 8; ++v) *reinterpret_cast<int4*>(c_row + v * 8) = make_int4(0, 0, 0, 0);
            }
            if (ok && row_ok) {
#pragma unroll
                for (int v = 0; v < kCols / 8; ++v) {
                    int4 out;
                    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(sum[v * 8 + 2 * i], sum[v * 8 + 2 * i + 1]);
                    *reinterpret_cast<int4*>(c_row + v * 8) = out;
                }
            }
        }
    }

    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

// ---------------------------------------------------------------- host side
// ==================================================================== e4m3 with hardware block scaling (128 x 256 tiles)
// For scales that are exact powers of two the tensor core applies them itself (tcgen05.mma kind::mxf8f6f4.block_scale,
// UE8M0 scale factors in tensor memory), so a tile accumulates over ALL of K in tensor memory and the epilogue runs once
// per tile instead of once per k-block. Roles: TMA producer, MMA issuer, eight epilogue warps (two per lane quarter, 128
// columns each), four scale warps (one per lane quarter). Per k-block of 128 a scale warp writes the slot of that
// pipeline stage in tensor memory: 4 columns for the rows of A (1x128 scales: all four 32-wide slices share the byte)
// and 8 columns for the 256 columns of B (128x128 scales: two bytes per k-block, replicated); `full[s]` collects the
// producer's bytes and the four scale warps, `empty[s]` (an MMA commit) frees both the shared-memory stage and its
// scale slot. The scale bytes of a tile are staged in shared memory one tile ahead, so the feed never waits for memory.
// The accumulator (256 columns) is single-buffered: tensor memory has 512 columns and the scale slots need their own.
struct MxCfg {
    static constexpr int BN = 256, BK = 128, UMMA_K = 32;
    static constexpr int kEpiWarps = 8, kSfWarps = 4;
    static constexpr int kThreads = (2 + kEpiWarps + kSfWarps) * 32;
    static constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
    static constexpr int kStages = 4;
    static constexpr int kSfCols = 16;                 // columns per scale slot: 4 (A) + 8 (B), padded to a store of 16
    static constexpr int kSfBase = BN;                 // first scale column behind the accumulator
    static constexpr int kTmemCols = 512;
    static constexpr int kMaxKb = 64;                  // k-blocks whose scale bytes fit the staging area (K <= 8192)
    static constexpr int kSfPitch = BM + 16;           // per k-block: 128 bytes for the rows of A, 2 for B
    static constexpr int kSfStage = kMaxKb * kSfPitch;
    static constexpr int kBarBytes = (2 * kStages + 2) * 8 + 16;
    static constexpr int kSmem = kStages * STAGE + 2 * kSfStage + kBarBytes + 1024;
};

__device__ __forceinline__ uint32_t ue8m0_of(float scale) { return (__float_as_uint(scale) >> 23) & 0xffu; }

__global__ void __launch_bounds__(MxCfg::kThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using C = MxCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sf_stage = smem + C::kStages * C::STAGE;                       // [2][kMaxKb][kSfPitch]
    uint64_t* full = reinterpret_cast<uint64_t*>(sf_stage + 2 * C::kSfStage);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);

    const int warp = warp_id(), lane = lane_id();
    PipeCtx pc{p.error, globaltimer_ns() + p.timeout_ns};

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full + s, 1 + C::kSfWarps);      // the producer's arrival (+ bytes) and one arrival per scale warp
            mbar_init(empty + s, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, C::kEpiWarps);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            Scheduler sched(p, C::BN, BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
                const int b_row = t.g * p.N + t.n0;
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    mbar_arrive_expect_tx(full + s, C::STAGE);
                    tma_load_2d(sa, &map_a, kb * C::BK, t.m0, full + s);
                    tma_load_2d(sa + C::A_BYTES, &map_b, kb * C::BK, b_row, full + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            Scheduler sched(p, C::BN, BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
                if (!(ok = pipe_wait(pc, tmem_empty, acc_ph ^ 1))) break;
                tc_fence_after();
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, full + s, ph))) break;
                    tc_fence_after();
                    const uint8_t* sa = smem + s * C::STAGE;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::A_BYTES);
                    const uint32_t sfa = tmem_base + C::kSfBase + s * C::kSfCols, sfb = sfa + 4;
#pragma unroll
                    for (int k = 0; k < C::BK / C::UMMA_K; ++k)
                        umma_mx(tmem_base, da + 2 * k, db + 2 * k, make_idesc_mx(BM, C::BN, static_cast<uint32_t>(k)),
                                (kb != t.kb0 || k != 0) ? 1u : 0u, sfa, sfb);
                    umma_commit(empty + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                umma_commit(tmem_full);
                acc_ph ^= 1;
            }
        }
    } else if (warp < 2 + C::kEpiWarps) {
        // ------------------------------------------------------------ epilogue warps: once per tile
        const int quarter = warp & 3;
        const int half = (warp - 2) / 4;               // which 128 of the 256 columns
        Scheduler sched(p, C::BN, BM, C::BK);
        Tile t;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int ti = blockIdx.x; ok && sched.get(ti, t); ti += gridDim.x) {
            const int row = t.m0 + quarter * 32 + lane;
            const bool row_ok = row < t.m_end && row < p.M;
            const bool zero_row = !row_ok && p.zero_gap && row < p.M;
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
            __nv_bfloat16* c_row = p.C + static_cast<int64_t>(row) * p.ldc + t.n0 + half * 128;
            if (!(ok = pipe_wait(pc, tmem_full, acc_ph))) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + c * 32, r);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        int4 out;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                        *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = out;
                    }
                } else if (zero_row) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = make_int4(0, 0, 0, 0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty);
            acc_ph ^= 1;
        }
    } else {
        // ------------------------------------------------------------ scale warps
        const int quarter = warp & 3;
        const int sf_tid = (warp - 2 - C::kEpiWarps) * 32 + lane;      // 0..127 = the row of the tile this thread stages
        const int kblocks = p.K / 128;
        Scheduler sched(p, C::BN, BM, C::BK);
        Tile t, nxt;
        auto stage_tile = [&](const Tile& tt, uint8_t* dst) {
            const int row = tt.m0 + sf_tid;
            const bool valid = row < tt.m_end && row < p.M;
            const float* src = p.sfa + static_cast<int64_t>(valid ? row : 0) * p.sfa_row_stride;
            for (int kb = tt.kb0; kb < tt.kb1; ++kb)
                dst[(kb - tt.kb0) * C::kSfPitch + sf_tid] = static_cast<uint8_t>(valid ? ue8m0_of(src[static_cast<int64_t>(kb) * p.sfa_k_stride]) : 127u);
            const float* srcb = p.sfb + (static_cast<int64_t>(tt.g) * (p.N / 128) + tt.n0 / 128) * kblocks;
            for (int i = sf_tid; i < 2 * (tt.kb1 - tt.kb0); i += C::kSfWarps * 32) {
                const int h = i & 1, kb = tt.kb0 + (i >> 1);
                dst[(kb - tt.kb0) * C::kSfPitch + BM + h] = static_cast<uint8_t>(ue8m0_of(srcb[static_cast<int64_t>(h) * kblocks + kb]));
            }
        };
        auto sf_barrier = [&]() { asm volatile("bar.sync 3, %0;" ::"r"(C::kSfWarps * 32) : "memory"); };
        int s = 0, buf = 0;
        uint32_t ph = 0;
        bool ok = true;
        bool have = sched.get(blockIdx.x, t);
        if (have) stage_tile(t, sf_stage);
        sf_barrier();
        for (int ti = blockIdx.x; ok && have; ti += gridDim.x) {
            const bool have_next = sched.get(ti + gridDim.x, nxt);
            if (have_next) stage_tile(nxt, sf_stage + (buf ^ 1) * C::kSfStage);      // one tile ahead
            const uint8_t* mine = sf_stage + buf * C::kSfStage;
            // two k-blocks per round: the wait for the tensor-memory stores (a few hundred cycles) is paid once per round,
            // otherwise a scale warp, which sees every k-block, could not keep up with the tensor pipe
            for (int kb = t.kb0; ok && kb < t.kb1; kb += 2) {
                const int n = min(2, t.kb1 - kb);
                int sj[2];
                for (int j = 0; j < n; ++j) {
                    sj[j] = s;
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                tc_fence_after();
                for (int j = 0; j < n; ++j) {
                    const uint8_t* src = mine + (kb + j - t.kb0) * C::kSfPitch;
                    uint32_t v[16];
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = static_cast<uint32_t>(src[lane + 32 * i]) * 0x01010101u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t b = static_cast<uint32_t>(src[BM + h]) * 0x01010101u;
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[4 + 4 * h + i] = b;
                    }
#pragma unroll
                    for (int i = 12; i < 16; ++i) v[i] = 0u;
                    tmem_st_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + C::kSfBase + sj[j] * C::kSfCols, v);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    for (int j = 0; j < n; ++j) {
                        mbar_arrive(full + sj[j]);
                    }
                }
            }
            sf_barrier();       // the next tile's bytes are complete; nobody reads this tile's any more
            buf ^= 1;
            t = nxt;
            have = have_next;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ==================================================================== e4m3 with hardware block scaling on CTA pairs (256 x 256 tiles)
// gemm_mx_kernel's scheme on the CTA-pair division of labour of gemm_pair_kernel: CTA r of the pair loads rows
// [128 r, 128 r + 128) of the A tile and of the B tile (32 KB per k-block and CTA instead of 48 KB: the block-scaled
// kernel on lone CTAs is bound by exactly this traffic), the leader issues tcgen05.mma.cta_group::2 with M = 256, each
// CTA's scale warps write the factors of its own 128 rows of A and of all 256 columns of B into its own tensor memory,
// each CTA's epilogue warps drain its 128 accumulator rows once per tile. `full` lives in the leader and collects the
// bytes of both CTAs and the eight scale warps of the pair; one multicast commit frees a stage (and its scale slot) in
// both CTAs; the leader's `tmem_empty` collects the epilogue warps of both.
struct MxPairCfg {
    static constexpr int BN = 256, BK = 128, UMMA_K = 32;
    static constexpr int kEpiWarps = 8, kSfWarps = 4;
    static constexpr int kThreads = (2 + kEpiWarps + kSfWarps) * 32;
    static constexpr int A_BYTES = BM * 128, B_BYTES = (BN / 2) * 128, STAGE = A_BYTES + B_BYTES;
    static constexpr int kStages = 6;
    static constexpr int kSfCols = 16, kSfBase = BN, kTmemCols = 512;
    static constexpr int kMaxKb = 64;
    static constexpr int kSfPitch = BM + 16;
    static constexpr int kSfStage = kMaxKb * kSfPitch;
    static constexpr int kBarBytes = (2 * kStages + 2) * 8 + 16;
    static constexpr int kSmem = kStages * STAGE + 2 * kSfStage + kBarBytes + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MxPairCfg::kThreads, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using C = MxPairCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sf_stage = smem + C::kStages * C::STAGE;
    uint64_t* full = reinterpret_cast<uint64_t*>(sf_stage + 2 * C::kSfStage);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);

    const int warp = warp_id(), lane = lane_id();
    const uint32_t cta = cluster_ctarank();
    const bool leader = cta == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    PipeCtx pc{p.error, globaltimer_ns() + p.timeout_ns};

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full + s, 1 + 2 * C::kSfWarps);
            mbar_init(empty + s, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 2 * C::kEpiWarps);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, C::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                const int b_row = t.g * p.N + t.n0 + static_cast<int>(cta) * (C::BN / 2);
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * C::STAGE;
                    if (leader) mbar_arrive_expect_tx(full + s, 2 * C::STAGE);
                    const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                    tma_load_2d_pair(sa, &map_a, kb * C::BK, t.m0 + static_cast<int>(cta) * BM, bar);
                    tma_load_2d_pair(sa + C::A_BYTES, &map_b, kb * C::BK, b_row, bar);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            Scheduler sched(p, C::BN, 2 * BM, C::BK);
            Tile t;
            int s = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
                if (!(ok = pipe_wait(pc, tmem_empty, acc_ph ^ 1))) break;
                tc_fence_after();
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!(ok = pipe_wait(pc, full + s, ph))) break;
                    tc_fence_after();
                    const uint8_t* sa = smem + s * C::STAGE;
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + C::A_BYTES);
                    const uint32_t sfa = tmem_base + C::kSfBase + s * C::kSfCols, sfb = sfa + 4;
#pragma unroll
                    for (int k = 0; k < C::BK / C::UMMA_K; ++k)
                        umma_mx_pair(tmem_base, da + 2 * k, db + 2 * k, make_idesc_mx(2 * BM, C::BN, static_cast<uint32_t>(k)),
                                     (kb != t.kb0 || k != 0) ? 1u : 0u, sfa, sfb);
                    umma_commit_pair(empty + s);
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(tmem_full);
                acc_ph ^= 1;
            }
        }
    } else if (warp < 2 + C::kEpiWarps) {
        // ------------------------------------------------------------ epilogue warps (both CTAs, own 128 rows), once per tile
        const int quarter = warp & 3;
        const int half = (warp - 2) / 4;
        Scheduler sched(p, C::BN, 2 * BM, C::BK);
        Tile t;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int ti = pair; ok && sched.get(ti, t); ti += num_pairs) {
            const int row = t.m0 + static_cast<int>(cta) * BM + quarter * 32 + lane;
            const bool row_ok = row < t.m_end && row < p.M;
            const bool zero_row = !row_ok && p.zero_gap && row < p.M && row < align_up(t.m_end, p.group_alignment);
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
            __nv_bfloat16* c_row = p.C + static_cast<int64_t>(row) * p.ldc + t.n0 + half * 128;
            if (!(ok = pipe_wait(pc, tmem_full, acc_ph))) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + c * 32, r);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        int4 out;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                        *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = out;
                    }
                } else if (zero_row) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) *reinterpret_cast<int4*>(c_row + c * 32 + v * 8) = make_int4(0, 0, 0, 0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty), 0));
            acc_ph ^= 1;
        }
    } else {
        // ------------------------------------------------------------ scale warps (both CTAs)
        const int quarter = warp & 3;
        const int sf_tid = (warp - 2 - C::kEpiWarps) * 32 + lane;
        const int kblocks = p.K / 128;
        Scheduler sched(p, C::BN, 2 * BM, C::BK);
        Tile t, nxt;
        auto stage_tile = [&](const Tile& tt, uint8_t* dst) {
            const int row = tt.m0 + static_cast<int>(cta) * BM + sf_tid;
            const bool valid = row < tt.m_end && row < p.M;
            const float* src = p.sfa + static_cast<int64_t>(valid ? row : 0) * p.sfa_row_stride;
            for (int kb = tt.kb0; kb < tt.kb1; ++kb)
                dst[(kb - tt.kb0) * C::kSfPitch + sf_tid] = static_cast<uint8_t>(valid ? ue8m0_of(src[static_cast<int64_t>(kb) * p.sfa_k_stride]) : 127u);
            const float* srcb = p.sfb + (static_cast<int64_t>(tt.g) * (p.N / 128) + tt.n0 / 128) * kblocks;
            for (int i = sf_tid; i < 2 * (tt.kb1 - tt.kb0); i += C::kSfWarps * 32) {
                const int h = i & 1, kb = tt.kb0 + (i >> 1);
                dst[(kb - tt.kb0) * C::kSfPitch + BM + h] = static_cast<uint8_t>(ue8m0_of(srcb[static_cast<int64_t>(h) * kblocks + kb]));
            }
        };
        auto sf_barrier = [&]() { asm volatile("bar.sync 3, %0;" ::"r"(C::kSfWarps * 32) : "memory"); };
        int s = 0, buf = 0;
        uint32_t ph = 0;
        bool ok = true;
        bool have = sched.get(pair, t);
        if (have) stage_tile(t, sf_stage);
        sf_barrier();
        for (int ti = pair; ok && have; ti += num_pairs) {
            const bool have_next = sched.get(ti + num_pairs, nxt);
            if (have_next) stage_tile(nxt, sf_stage + (buf ^ 1) * C::kSfStage);
            const uint8_t* mine = sf_stage + buf * C::kSfStage;
            // two k-blocks per round: the wait for the tensor-memory stores (a few hundred cycles) is paid once per round,
            // otherwise a scale warp, which sees every k-block, could not keep up with the tensor pipe
            for (int kb = t.kb0; ok && kb < t.kb1; kb += 2) {
                const int n = min(2, t.kb1 - kb);
                int sj[2];
                for (int j = 0; j < n; ++j) {
                    sj[j] = s;
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    if (++s == C::kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                tc_fence_after();
                for (int j = 0; j < n; ++j) {
                    const uint8_t* src = mine + (kb + j - t.kb0) * C::kSfPitch;
                    uint32_t v[16];
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = static_cast<uint32_t>(src[lane + 32 * i]) * 0x01010101u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t b = static_cast<uint32_t>(src[BM + h]) * 0x01010101u;
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[4 + 4 * h + i] = b;
                    }
#pragma unroll
                    for (int i = 12; i < 16; ++i) v[i] = 0u;
                    tmem_st_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + C::kSfBase + sj[j] * C::kSfCols, v);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    for (int j = 0; j < n; ++j) {
                        // (the stores are complete: tcgen05.wait::st above; the arrival only has to get there)
                        if (leader) mbar_arrive(full + sj[j]);
                        else mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(full + sj[j]), 0));
                    }
                }
            }
            sf_barrier();
            buf ^= 1;
            t = nxt;
            have = have_next;
        }
    }

    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

}  // namespace

// 2-D K-major tensor map: `rows` x `cols` elements of `elem_bytes`, row pitch `row_stride_bytes`,
// box = `box_rows` x (128 / elem_bytes) elements, 128-byte swizzle.
bool make_kmajor_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                     uint32_t box_rows) {
    EncodeFn encode = get_encode_fn();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dtype = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    return encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool kFp8>
static cudaError_t launch_cfg(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, int num_sms, cudaStream_t stream) {
    using C = Cfg<BN, kFp8>;
    cudaError_t err = cudaFuncSetAttribute(gemm_kernel<BN, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);
    if (err != cudaSuccess) return err;
    gemm_kernel<BN, kFp8><<<num_sms, C::kThreads, C::kSmem, stream>>>(map_a, map_b, p);
    return cudaGetLastError();
}

cudaError_t launch_gemm(const GemmParams& p, const void* a, int64_t a_row_stride_bytes, const void* b, int64_t b_row_stride_bytes,
                        bool fp8, int num_sms, cudaStream_t stream) {
    const int elem = fp8 ? 1 : 2;
    // bf16 with 256-wide tiles runs on CTA pairs (EP_GEMM_CTA_PAIR=0 keeps one CTA per tile); a pair needs two SMs.
    // e4m3 on CTA pairs is opt-in (EP_GEMM_FP8_PAIR=1): with software block scaling the 256 x 256 tile halves the
    // shared-memory fill per flop, but only two accumulator passes fit into tensor memory and the drain of a pass
    // (64 columns per epilogue thread) then sets the pace: 0.94 PFLOP/s measured against 1.3 with 128 x 128 tiles and
    // four passes in flight.
    const char* pair_env = std::getenv("EP_GEMM_CTA_PAIR");
    const char* fp8_pair_env = std::getenv("EP_GEMM_FP8_PAIR");
    const bool pair_enabled = fp8 ? (fp8_pair_env != nullptr && fp8_pair_env[0] == '1') : (pair_env == nullptr || pair_env[0] != '0');
    const bool use_pair = p.N % 256 == 0 && pair_enabled && num_sms >= 2;
    const int bn = fp8 ? (use_pair ? 256 : 128) : ((p.N % 256 == 0) ? 256 : 128);
    const int bk = fp8 ? 128 : 64;
    if (p.N % bn != 0 || p.K % bk != 0 || p.M <= 0) return cudaErrorInvalidValue;
    if (p.k_grouped && (fp8 || p.group_end == nullptr || p.group_alignment % bk != 0)) return cudaErrorInvalidValue;
    CUtensorMap map_a, map_b;
    if (!make_kmajor_map(&map_a, a, elem, static_cast<uint64_t>(p.M), static_cast<uint64_t>(p.K), static_cast<uint64_t>(a_row_stride_bytes), BM) ||
        !make_kmajor_map(&map_b, b, elem, static_cast<uint64_t>(p.num_groups) * p.N, static_cast<uint64_t>(p.K),
                         static_cast<uint64_t>(b_row_stride_bytes), static_cast<uint32_t>(use_pair ? bn / 2 : bn)))
        return cudaErrorInvalidValue;
    // e4m3 with power-of-two scales: the block-scaled instruction kind (EP_GEMM_FP8_MX=0 keeps the software scaling)
    const char* mx_env = std::getenv("EP_GEMM_FP8_MX");
    const bool mx_enabled = mx_env == nullptr || mx_env[0] != '0';
    if (fp8 && p.scales_pow2 && mx_enabled && !use_pair && p.N % 256 == 0 && p.K / 128 <= MxCfg::kMaxKb && !p.k_grouped) {
        // CTA pairs (EP_GEMM_FP8_MX_PAIR=1): 256 x 256 tiles, each CTA loads 128 rows of A and 128 of B. Opt-in: measured
        // no faster than lone CTAs (2.21 against 2.16 PFLOP/s), so the fill of shared memory from L2 is not what limits
        // the lone-CTA kernel; per k-block a CTA's shared memory takes 48 KB from TMA and hands 48 KB to the tensor
        // core in 541 tensor-pipe cycles either way, more than its 128 bytes per cycle.
        const char* mx_pair_env = std::getenv("EP_GEMM_FP8_MX_PAIR");
        const bool mx_pair = mx_pair_env != nullptr && mx_pair_env[0] == '1';
        if (mx_pair && num_sms >= 2) {
            CUtensorMap map_b128;
            if (!make_kmajor_map(&map_b128, b, elem, static_cast<uint64_t>(p.num_groups) * p.N, static_cast<uint64_t>(p.K),
                                 static_cast<uint64_t>(b_row_stride_bytes), 128))
                return cudaErrorInvalidValue;
            cudaError_t err = cudaFuncSetAttribute(gemm_mx_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MxPairCfg::kSmem);
            if (err != cudaSuccess) return err;
            gemm_mx_pair_kernel<<<num_sms & ~1, MxPairCfg::kThreads, MxPairCfg::kSmem, stream>>>(map_a, map_b128, p);
            return cudaGetLastError();
        }
        CUtensorMap map_b256;
        if (!make_kmajor_map(&map_b256, b, elem, static_cast<uint64_t>(p.num_groups) * p.N, static_cast<uint64_t>(p.K),
                             static_cast<uint64_t>(b_row_stride_bytes), 256))
            return cudaErrorInvalidValue;
        cudaError_t err = cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MxCfg::kSmem);
        if (err != cudaSuccess) return err;
        gemm_mx_kernel<<<num_sms, MxCfg::kThreads, MxCfg::kSmem, stream>>>(map_a, map_b256, p);
        return cudaGetLastError();
    }
    if (fp8 && use_pair) {
        cudaError_t err = cudaFuncSetAttribute(gemm_pair_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairFp8Cfg::kSmem);
        if (err != cudaSuccess) return err;
        gemm_pair_fp8_kernel<<<num_sms & ~1, PairFp8Cfg::kThreads, PairFp8Cfg::kSmem, stream>>>(map_a, map_b, p);
        return cudaGetLastError();
    }
    if (fp8) return launch_cfg<128, true>(map_a, map_b, p, num_sms, stream);
    if (bn == 256 && use_pair) {
        cudaError_t err = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmem);
        if (err != cudaSuccess) return err;
        gemm_pair_kernel<<<num_sms & ~1, PairCfg::kThreads, PairCfg::kSmem, stream>>>(map_a, map_b, p);
        return cudaGetLastError();
    }
    if (bn == 256) return launch_cfg<256, false>(map_a, map_b, p, num_sms, stream);
    return launch_cfg<128, false>(map_a, map_b, p, num_sms, stream);
}

}  // namespace gemm
}  // namespace ep
