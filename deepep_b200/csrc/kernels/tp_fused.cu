// Tensor-parallel GEMMs fused with their collective, one kernel each (bf16, sm_100a):
//
//   all-gather -> GEMM    C[R*Ml, N] = gather_r(A_r[Ml, K]) * B[N, K]^T
//       The shard reaches every peer's gather buffer in 128-row chunks with one arrival flag per
//       (source, chunk) at the peer, either from a few "comm" CTAs of this kernel (bulk copies over
//       NVLink, rows counted behind device-scope fences, the chunk's flag a system-scope release by
//       the thread that completes it) or, with no CTA spent on it, from the copy engines (two copies
//       per peer on side streams, the flags of a copy's chunks one batched stream write behind it;
//       issued by the host driver, which picks the form by the GEMM's length against its own cost).
//       The GEMM CTAs run the tcgen05 main loop; the TMA producer of a tile waits (bounded) for
//       the flag of the chunk it is about to read, so the math on early chunks overlaps the
//       transfer of late ones. Own rows are read straight from the input and go first.
//       All TMA loads read LOCAL memory (the input or the local gather buffer); none is multicast.
//
//   GEMM -> reduce-scatter    out[Ml, N] = sum_r (A_r[R*Ml, Kl] * B_r[N, Kl]^T)[rows of this rank]
//       Tiles are computed destination by destination (next rank first, own rows last). For a
//       peer's rows the epilogue converts the accumulator to bf16, stages it in shared memory and
//       bulk-stores it into slot [this rank] of the destination's partial buffer, then raises a
//       per-tile flag there. For the rank's own rows, which come last, the peers' partial tiles
//       have arrived by then: with up to four ranks the epilogue waits for their flags, adds them
//       to the fp32 accumulator in rank order and writes the final rows (no partial of its own, no
//       reduction pass); with more ranks the own rows go through the partial buffer as well and
//       every CTA reduces a share of the rank's tiles after its GEMM tiles.
//
// Both kernels walk their tiles in bands of eight row blocks with the row index fastest, so the
// tiles in flight share few operand blocks (L2 reuse).
//
// The reference has neither operator (its AGRS path is a copy-engine all-gather only, and
// reduce-scatter is listed as not implemented); the baseline to beat is NCCL all-gather /
// reduce-scatter followed / preceded by an unfused GEMM.
#include <cstdlib>

#include "gemm_api.hpp"
#include "gemm_sm100.cuh"
#include "tp_api.hpp"

namespace ep {
namespace gemm {

namespace {

constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;

__device__ __forceinline__ void init_pipeline(uint64_t* full, uint64_t* empty, uint64_t* tmem_full, uint64_t* tmem_empty, int stages,
                                              int epi_threads) {
    for (int s = 0; s < stages; ++s) {
        mbar_init(full + s, 1);
        mbar_init(empty + s, 1);
    }
    for (int a = 0; a < 2; ++a) {
        mbar_init(tmem_full + a, 1);
        mbar_init(tmem_empty + a, epi_threads);
    }
    fence_mbar_init();
}

// the MMA warp is the same for both operators: consume stages, accumulate one tile per accumulator
template <int kStages>
__device__ __forceinline__ void mma_role(const PipeCtx& pc, uint8_t* smem, uint64_t* full, uint64_t* empty, uint64_t* tmem_full,
                                         uint64_t* tmem_empty, uint32_t tmem_base, int num_tiles_mine, int num_kb) {
    constexpr uint32_t idesc = make_idesc<false>(BM, BN);
    int s = 0, acc = 0;
    uint32_t ph = 0, acc_ph = 0;
    for (int i = 0; i < num_tiles_mine; ++i) {
        if (!pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1)) return;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
            if (!pipe_wait(pc, full + s, ph)) return;
            tc_fence_after();
            const uint8_t* sa = smem + s * STAGE;
            const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma<false>(tmem_base + acc * BN, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            umma_commit(empty + s);
            if (++s == kStages) { s = 0; ph ^= 1; }
        }
        umma_commit(tmem_full + acc);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
    }
}

// CTA-pair form (leader CTA only): 256-row tiles, stages of A_BYTES + B_BYTES / 2 per CTA, barriers of both CTAs
// released by multicast commits (see gemm_sm100.cuh)
constexpr int STAGE_PAIR = A_BYTES + B_BYTES / 2;
template <int kStages>
__device__ __forceinline__ void mma_role_pair(const PipeCtx& pc, uint8_t* smem, uint64_t* full, uint64_t* empty, uint64_t* tmem_full,
                                              uint64_t* tmem_empty, uint32_t tmem_base, int num_tiles_mine, int num_kb) {
    constexpr uint32_t idesc = make_idesc<false>(2 * BM, BN);
    int s = 0, acc = 0;
    uint32_t ph = 0, acc_ph = 0;
    for (int i = 0; i < num_tiles_mine; ++i) {
        if (!pipe_wait(pc, tmem_empty + acc, acc_ph ^ 1)) return;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
            if (!pipe_wait(pc, full + s, ph)) return;
            tc_fence_after();
            const uint8_t* sa = smem + s * STAGE_PAIR;
            const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_pair_bf16(tmem_base + acc * BN, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            umma_commit_pair(empty + s);
            if (++s == kStages) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(tmem_full + acc);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
    }
}

__device__ __forceinline__ int tiles_of(int total, int first, int stride) {
    return total > first ? (total - first + stride - 1) / stride : 0;
}

// ==================================================================== all-gather -> GEMM
constexpr int kAgThreads = 6 * 32;
// kPair: GEMM CTAs work in clusters of two on two 128-row chunks and one 256-column block of B (cta_group::2)
template <bool kPair>
struct AgCfg {
    static constexpr int kStages = kPair ? 6 : 4;
    static constexpr int kStage = kPair ? STAGE_PAIR : STAGE;
    static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmem = kStages * kStage + kBarBytes + 1024;
};
constexpr int kAgSmem = AgCfg<false>::kSmem;   // both forms: 192 KB of stages
static_assert(AgCfg<true>::kSmem == AgCfg<false>::kSmem + 4 * 8, "the comm CTAs size their row buffers by kAgSmem");

// one launch may carry several virtual ranks (single-GPU emulation): CTAs [v * ctas_per_rank, ...) act as rank v
struct AgLaunch {
    int num_vranks, ctas_per_rank;
    AgGemmParams p[kTpMaxVRanks];
    CUtensorMap map_local[kTpMaxVRanks], map_gather[kTpMaxVRanks], map_b[kTpMaxVRanks];
};
struct RsLaunch {
    int num_vranks, ctas_per_rank;
    GemmRsParams p[kTpMaxVRanks];
    CUtensorMap map_a[kTpMaxVRanks], map_b[kTpMaxVRanks];
};

// Work items of a (rows x tiles_n) grid in bands of kBand rows: inside a band the row index runs fastest, so the CTAs at
// work at any one time share a few B column blocks and a few A row blocks, which then stay in L2 (with the column
// index fastest, every pass over one row block streams the whole of B, more than L2 holds, from memory again).
constexpr int kBand = 8;
__device__ __forceinline__ void band_order(int u, int rows, int tiles_n, int& m, int& n) {
    const int band = u / (kBand * tiles_n);
    const int g = min(kBand, rows - band * kBand);
    const int v = u - band * kBand * tiles_n;
    n = v / g;
    m = band * kBand + v % g;
}

template <bool kPair>
__global__ void __launch_bounds__(kAgThreads, 1) ag_gemm_kernel(const __grid_constant__ AgLaunch L) {
    constexpr int kAgStages = AgCfg<kPair>::kStages;
    constexpr int kStageBytes = AgCfg<kPair>::kStage;
    const int vr = blockIdx.x / L.ctas_per_rank;
    const int bid = blockIdx.x % L.ctas_per_rank, nctas = L.ctas_per_rank;
    const AgGemmParams& p = L.p[vr];
    const CUtensorMap& map_local = L.map_local[vr];
    const CUtensorMap& map_gather = L.map_gather[vr];
    const CUtensorMap& map_b = L.map_b[vr];
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int warp = warp_id(), lane = lane_id();
    const CommCtx& c = p.c;
    const int R = c.num_ranks, Ml = p.rows_per_rank, K = p.K;
    const int chunks = Ml / BM;
    const WaitCtx w = make_wait_ctx(c);

    if (bid < p.num_comm_ctas) {
        // ------------------------------------------------------------ comm CTAs: push the local shard to every peer
        // unit = (chunk, peer, row): one warp moves one row (K * 2 bytes) through its shared-memory buffer
        const int row_bytes = K * 2;
        const int stage = align_up(row_bytes, 128) + 16;
        uint8_t* buf = smem + static_cast<size_t>(warp) * stage;
        uint64_t* bar = reinterpret_cast<uint64_t*>(buf + align_up(row_bytes, 128));
        if (lane == 0) {
            mbar_init(bar, 1);
            fence_mbar_init();
        }
        __syncwarp();
        int* done = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsTpOffsetBytes);   // [chunks][R] rows landed, reset by the flag sender
        // Entry handshake: a peer's gather buffer half may only be overwritten once that peer has entered
        // this call (and so has finished the call that last read the half).
        if (warp == 0 && lane < R && lane != c.rank) {
            uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[lane]) + kCtlTileFlags + c.rank * 64 + 63;
            if (bid == 0) st_release_sys_u64(remote, pack_epoch(p.epoch, 0));
            const uint64_t* mine_flag = reinterpret_cast<const uint64_t*>(c.heap[c.rank]) + kCtlTileFlags + lane * 64 + 63;
            if (!bounded_wait(w, kStatusTileFlag, lane, 63, [&]() { return epoch_reached(ld_acquire_sys_u64(mine_flag), p.epoch); }))
                atomicExch(p.error, static_cast<int>(kStatusTileFlag));
        }
        __syncthreads();
        const int num_warps = kAgThreads / 32;
        const int workers = p.num_comm_ctas * num_warps;
        const int me = bid * num_warps + warp;
        uint32_t parity = 0;
        // Two buffers per warp; a buffer is reused once its store has READ it (wait_group.read), while rows are
        // counted as landed at least four rows late, once wait_group has confirmed their remote writes. The count is a
        // device-scope atomic behind a device-scope fence (all counting threads are on this GPU); only the thread that
        // completes a chunk pays the system-scope fence and release store that carry the chunk's rows to the peer
        // (a system-scope fence per row, tried in between, cost 20 % at TP8: 397 against 327 us). Several rows per lane
        // are therefore on the wire at any time and the NVLink round trip stays off the critical path.
        auto landed_row = [&](int chunk) {       // after a device-scope fence behind the row's wait_group
            const int old = atomicAdd(done + chunk * kMaxRanks + lane, 1);
            if (old == BM - 1) {
                done[chunk * kMaxRanks + lane] = 0;
                fence_acq_rel_sys();             // behind the other senders' rows, which their (fenced) adds announced
                uint64_t* flag = reinterpret_cast<uint64_t*>(c.heap[lane]) + kCtlTileFlags + c.rank * 64 + chunk;
                st_release_sys_u64(flag, pack_epoch(p.epoch, 1));
            }
        };
        const bool sender = lane < R && lane != c.rank;
        uint8_t* buf2[2] = {buf, buf + num_warps * stage};
        int it = 0, retired = 0;     // rows of this warp sent / counted as landed (row of iteration j = me + j * workers)
        // rows counted per fence: four where a warp has many rows; with few rows per warp (large TP degrees) batching
        // would hold every chunk's flag back until the warp is done (TP8: 8 rows per warp)
        const int rows_per_warp = ceil_div(Ml, workers);
        const int batch = rows_per_warp >= 32 ? 4 : (rows_per_warp >= 16 ? 2 : 1);
        for (int row = me; row < Ml && R > 1; row += workers, ++it) {
            uint8_t* cur = buf2[it & 1];
            bulk_wait_read<1>();        // the store that used this buffer two rows ago has read it
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, row_bytes);
                bulk_g2s(cur, p.a_local + static_cast<int64_t>(row) * p.a_stride_bytes, row_bytes, bar);
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, row);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) break;
            if (sender) {
                bulk_s2g(c.heap[lane] + p.off_gather + (static_cast<uint64_t>(c.rank) * Ml + row) * row_bytes, cur, row_bytes);
                bulk_commit();
                if (it - 3 - retired >= batch) {     // `batch` more rows are at least four stores old
                    bulk_wait<4>();
                    __threadfence();
                    for (; retired <= it - 4; ++retired) landed_row((me + retired * workers) / BM);
                }
            }
            __syncwarp();
        }
        if (sender && retired < it) {
            bulk_wait_all();
            __threadfence();
            for (; retired < it; ++retired) landed_row((me + retired * workers) / BM);
        }
        bulk_wait_all();
        return;
    }

    // ---------------------------------------------------------------- GEMM CTAs
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kAgStages * kStageBytes);
    uint64_t* empty = full + kAgStages;
    uint64_t* tmem_full = empty + kAgStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    PipeCtx pc{p.error, globaltimer_ns() + c.timeout_ns};
    const int num_kb = K / BK;
    const int tiles_n = p.N / BN;
    // pair: work item = (two consecutive entries of the arrival order, n block); CTA `cta` of the pair takes entry 2 * op + cta
    const uint32_t cta = kPair ? cluster_ctarank() : 0u;
    const int total_tiles = (kPair ? R * chunks / 2 : R * chunks) * tiles_n;
    const int first = kPair ? (bid - p.num_comm_ctas) >> 1 : bid - p.num_comm_ctas;
    const int stride = kPair ? (nctas - p.num_comm_ctas) >> 1 : nctas - p.num_comm_ctas;
    const int mine = tiles_of(total_tiles, first, stride);

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_local);
        prefetch_tensormap(&map_gather);
        prefetch_tensormap(&map_b);
        init_pipeline(full, empty, tmem_full, tmem_empty, kAgStages, kPair ? 8 * 32 : 4 * 32);
    }
    if (warp == 1) {
        if constexpr (kPair) {
            tmem_alloc_pair(tmem_slot, 2 * BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 2 * BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if constexpr (kPair) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // tile t -> (order index o, n block): o walks own rows first, then chunk by chunk over the sources rank+1, rank+2, ...
    auto decode = [&](int t, int& src, int& chunk, int& n0) {
        int oi, ni;
        band_order(t, total_tiles / tiles_n, tiles_n, oi, ni);
        const int o = kPair ? 2 * oi + static_cast<int>(cta) : oi;
        n0 = ni * BN;
        if (o < chunks) {
            src = c.rank;
            chunk = o;
        } else {
            const int q = o - chunks;
            chunk = q / (R - 1);
            src = (c.rank + 1 + q % (R - 1)) % R;
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = first; ok && t < total_tiles; t += stride) {
                int src, chunk, n0;
                decode(t, src, chunk, n0);
                if (src != c.rank) {
                    const uint64_t* flag = reinterpret_cast<const uint64_t*>(c.heap[c.rank]) + kCtlTileFlags + src * 64 + chunk;
                    ok = bounded_wait(w, kStatusTileFlag, src, chunk, [&]() { return epoch_reached(ld_acquire_sys_u64(flag), p.epoch); });
                    if (!ok) {
                        atomicExch(p.error, static_cast<int>(kStatusTileFlag));
                        break;
                    }
                }
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * kStageBytes;
                    if constexpr (kPair) {
                        if (cta == 0) mbar_arrive_expect_tx(full + s, 2 * kStageBytes);
                        const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                        if (src == c.rank) tma_load_2d_pair(sa, &map_local, kb * BK, chunk * BM, bar);
                        else tma_load_2d_pair(sa, &map_gather, kb * BK, src * Ml + chunk * BM, bar);
                        tma_load_2d_pair(sa + A_BYTES, &map_b, kb * BK, n0 + static_cast<int>(cta) * (BN / 2), bar);
                    } else {
                        mbar_arrive_expect_tx(full + s, STAGE);
                        if (src == c.rank) tma_load_2d(sa, &map_local, kb * BK, chunk * BM, full + s);
                        else tma_load_2d(sa, &map_gather, kb * BK, src * Ml + chunk * BM, full + s);
                        tma_load_2d(sa + A_BYTES, &map_b, kb * BK, n0, full + s);
                    }
                    if (++s == kAgStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if constexpr (kPair) {
            if (cta == 0 && lane == 0) mma_role_pair<kAgStages>(pc, smem, full, empty, tmem_full, tmem_empty, tmem_base, mine, num_kb);
        } else {
            if (lane == 0) mma_role<kAgStages>(pc, smem, full, empty, tmem_full, tmem_empty, tmem_base, mine, num_kb);
        }
    } else {
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int t = first; t < total_tiles; t += stride) {
            int src, chunk, n0;
            decode(t, src, chunk, n0);
            const int row = src * Ml + chunk * BM + quarter * 32 + lane;
            if (!pipe_wait(pc, tmem_full + acc, acc_ph)) break;
            tc_fence_after();
            __nv_bfloat16* c_row = p.C + static_cast<int64_t>(row) * p.ldc + n0;
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + cc * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    int4 out;
                    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                    *reinterpret_cast<int4*>(c_row + cc * 32 + v * 8) = out;
                }
            }
            tc_fence_before();
            if constexpr (kPair) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
            else mbar_arrive(tmem_empty + acc);
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1;
        }
    }
    tc_fence_before();
    if constexpr (kPair) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, 2 * BN);
        else tmem_dealloc(tmem_base, 2 * BN);
    }
}

// ==================================================================== GEMM -> reduce-scatter
constexpr int kRsRowPitch = BN * 2 + 16;                       // padded rows: lanes of a warp fall into different banks
constexpr int kRsStageTile = BM * kRsRowPitch;                 // bf16 staging tile of the epilogue
constexpr int kRsThreads = 6 * 32;
// kPair: two CTAs of a cluster share a 256-row tile (tcgen05 cta_group::2): each loads its 128 rows of A and half of
// the B tile, four 32 KB stages instead of three 48 KB ones fit next to the staging tile.
template <bool kPair>
struct RsCfg {
    static constexpr int kStages = kPair ? 4 : 3;
    static constexpr int kStage = kPair ? STAGE_PAIR : STAGE;
    static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmem = kStages * kStage + kRsStageTile + kBarBytes + 1024;
};

template <bool kPair>
__global__ void __launch_bounds__(kRsThreads, 1) gemm_rs_kernel(const __grid_constant__ RsLaunch L) {
    constexpr int kRsStages = RsCfg<kPair>::kStages;
    constexpr int kStageBytes = RsCfg<kPair>::kStage;
    const int vr = blockIdx.x / L.ctas_per_rank;
    const int bid = blockIdx.x % L.ctas_per_rank, nctas = L.ctas_per_rank;
    const GemmRsParams& p = L.p[vr];
    const CUtensorMap& map_a = L.map_a[vr];
    const CUtensorMap& map_b = L.map_b[vr];
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* stage_tile = smem + kRsStages * kStageBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(stage_tile + kRsStageTile);
    uint64_t* empty = full + kRsStages;
    uint64_t* tmem_full = empty + kRsStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    const int warp = warp_id(), lane = lane_id();
    const CommCtx& c = p.c;
    const int R = c.num_ranks, Ml = p.rows_per_rank, N = p.N;
    const int chunks = Ml / BM, tiles_n = N / BN;
    const int tiles_per_dst = chunks * tiles_n;
    const int total_tiles = R * tiles_per_dst;
    const int num_kb = p.K / BK;
    const WaitCtx w = make_wait_ctx(c);
    PipeCtx pc{p.error, globaltimer_ns() + c.timeout_ns};
    // pair: the unit of work is a 256-row tile owned by CTAs (2j, 2j + 1); CTA `cta` computes chunk 2 * c + cta of it
    const uint32_t cta = kPair ? cluster_ctarank() : 0u;
    const int first = kPair ? bid >> 1 : bid, stride = kPair ? nctas >> 1 : nctas;
    const int work_per_dst = kPair ? tiles_per_dst / 2 : tiles_per_dst;
    const int total_work = R * work_per_dst;
    const int mine = tiles_of(total_work, first, stride);
    const int half = p.epoch & 1;
    const uint64_t part_off = p.off_partial[half], flag_off = p.off_flags[half];
    const bool fuse_own = p.fuse_own != 0;  // the epilogue of the own rows adds the peers' partial tiles itself

    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        init_pipeline(full, empty, tmem_full, tmem_empty, kRsStages, kPair ? 8 * 32 : 4 * 32);
    }
    if (warp == 1) {
        if constexpr (kPair) {
            tmem_alloc_pair(tmem_slot, 2 * BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 2 * BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if constexpr (kPair) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // work item t -> destination (next rank first, own rows last) and the 128-row tile this CTA computes of it
    auto decode = [&](int t, int& dst, int& local_tile) {
        dst = (c.rank + 1 + t / work_per_dst) % R;
        int mi, ni;
        band_order(t % work_per_dst, work_per_dst / tiles_n, tiles_n, mi, ni);
        local_tile = (kPair ? mi * 2 + static_cast<int>(cta) : mi) * tiles_n + ni;
    };

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = first; ok && t < total_work; t += stride) {
                int dst, lt;
                decode(t, dst, lt);
                const int m0 = dst * Ml + (lt / tiles_n) * BM, n0 = (lt % tiles_n) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = pipe_wait(pc, empty + s, ph ^ 1))) break;
                    uint8_t* sa = smem + s * kStageBytes;
                    if constexpr (kPair) {
                        if (cta == 0) mbar_arrive_expect_tx(full + s, 2 * kStageBytes);
                        const uint32_t bar = map_to_cta(smem_u32(full + s), 0);
                        tma_load_2d_pair(sa, &map_a, kb * BK, m0, bar);
                        tma_load_2d_pair(sa + A_BYTES, &map_b, kb * BK, n0 + static_cast<int>(cta) * (BN / 2), bar);
                    } else {
                        mbar_arrive_expect_tx(full + s, STAGE);
                        tma_load_2d(sa, &map_a, kb * BK, m0, full + s);
                        tma_load_2d(sa + A_BYTES, &map_b, kb * BK, n0, full + s);
                    }
                    if (++s == kRsStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if constexpr (kPair) {
            if (cta == 0 && lane == 0) mma_role_pair<kRsStages>(pc, smem, full, empty, tmem_full, tmem_empty, tmem_base, mine, num_kb);
        } else {
            if (lane == 0) mma_role<kRsStages>(pc, smem, full, empty, tmem_full, tmem_empty, tmem_base, mine, num_kb);
        }
    } else {
        // epilogue: accumulator -> bf16 -> staging tile -> bulk stores into the destination's partial slot -> flag.
        // This rank's own rows come last; by then the peers' partial tiles for them have long arrived (every rank
        // starts with the rows of the rank behind it). With up to four ranks the epilogue adds them to the fp32
        // accumulator and writes the final rows: no partial tile of its own to store and re-read, no reduction pass
        // after the GEMM (887 -> 797 us at TP2). With more ranks that epilogue would read seven partial tiles per own
        // tile in dependent rounds while the accumulator waits (481 us against 386 us for the baseline at TP8), so the
        // own rows go to the local partial slot like any other and a reduction pass follows the GEMM.
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_ph = 0;
        uint64_t* prev_flag = nullptr;
        const uint64_t* my_flags = reinterpret_cast<const uint64_t*>(c.heap[c.rank] + flag_off);
        const uint8_t* my_part = c.heap[c.rank] + part_off;
        const uint64_t target = static_cast<uint64_t>(p.flag_target);
        const uint64_t slot_bytes = static_cast<uint64_t>(Ml) * N * 2;
        for (int t = first; t < total_work; t += stride) {
            int dst, lt;
            decode(t, dst, lt);
            const int local_m0 = (lt / tiles_n) * BM, n0 = (lt % tiles_n) * BN;
            const bool own = fuse_own && dst == c.rank;
            if (own) {
                // Nothing of this rank may still be owed to a peer while it waits for the peers: the arrival of the
                // previous tile, normally raised one tile late, goes out first (two ranks that each held back the
                // tile the other one is waiting for would wait for each other).
                if (prev_flag != nullptr) {
                    bulk_wait_all();
                    __syncwarp();
                    if (lane == 0) red_add_release_sys_u64(prev_flag, 1);
                    prev_flag = nullptr;
                }
                bool arrived = true;
                if (lane < R && lane != c.rank) {
                    const uint64_t* flag = my_flags + static_cast<uint64_t>(lane) * tiles_per_dst + lt;
                    arrived = bounded_wait(w, kStatusTileFlag, lane, lt, [&]() { return ld_acquire_sys_u64(flag) >= target; });
                }
                if (!__all_sync(0xffffffffu, arrived) && lane == 0) atomicExch(p.error, static_cast<int>(kStatusTileFlag));
                __syncwarp();
            }
            if (!pipe_wait(pc, tmem_full + acc, acc_ph)) break;
            tc_fence_after();
            // (the previous tile's bulk store of this lane has completed: it is waited for right after it is issued)
            const int r_in_tile = quarter * 32 + lane;
            __nv_bfloat16* srow = reinterpret_cast<__nv_bfloat16*>(stage_tile + static_cast<size_t>(r_in_tile) * kRsRowPitch);
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + cc * 32, r);
                tmem_ld_wait();
                if (own) {
                    // 64 bytes of every peer's partial row, two peers (eight 16-byte loads) in flight per lane
                    const uint8_t* base = my_part + ((static_cast<uint64_t>(local_m0) + r_in_tile) * N + n0 + cc * 32) * 2;
#pragma unroll 1
                    for (int s0 = 0; s0 < R; s0 += 2) {
                        int4 pr[2][4];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int src = s0 + u;
                            if (src < R && src != c.rank) {
#pragma unroll
                                for (int v = 0; v < 4; ++v) pr[u][v] = ld_nc_int4(base + src * slot_bytes + v * 16);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int src = s0 + u;
                            if (src < R && src != c.rank) {
#pragma unroll
                                for (int v = 0; v < 4; ++v) {
                                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&pr[u][v]);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        const float2 f = __bfloat1622float2(h2[i]);
                                        r[v * 8 + 2 * i] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * i]) + f.x);
                                        r[v * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * i + 1]) + f.y);
                                    }
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    int4 out;
                    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o2[i] = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * i]), __uint_as_float(r[v * 8 + 2 * i + 1]));
                    *reinterpret_cast<int4*>(srow + cc * 32 + v * 8) = out;
                }
            }
            tc_fence_before();
            if constexpr (kPair) mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty + acc), 0));
            else mbar_arrive(tmem_empty + acc);
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1;
            fence_proxy_async_smem();
            __syncwarp();
            uint8_t* dst_base = own ? reinterpret_cast<uint8_t*>(p.out) + (static_cast<uint64_t>(local_m0 + r_in_tile) * p.ldo + n0) * 2
                                    : c.heap[dst] + part_off + ((static_cast<uint64_t>(c.rank) * Ml + local_m0 + r_in_tile) * N + n0) * 2;
            bulk_s2g(dst_base, srow, BN * 2);
            bulk_commit();
            // The flag of the PREVIOUS tile is raised now (its stores have had a whole tile time to complete); this
            // tile's store only has to have read the staging row before the next tile overwrites it.
            bulk_wait<1>();
            if (prev_flag != nullptr) {
                // every lane's store of the previous tile is complete (wait_group above); the warp barrier collects
                // them behind the one release add of the tile
                __syncwarp();
                if (lane == 0) red_add_release_sys_u64(prev_flag, 1);
            }
            prev_flag = own ? nullptr : reinterpret_cast<uint64_t*>(c.heap[dst] + flag_off) + static_cast<uint64_t>(c.rank) * tiles_per_dst + lt;
            bulk_wait_read_all();
            __syncwarp();
        }
        bulk_wait_all();
        if (prev_flag != nullptr) {
            __syncwarp();
            // one arrival per epilogue warp on the tile's flag word: the reducer waits for 4 arrivals per call
            if (lane == 0) red_add_release_sys_u64(prev_flag, 1);
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before();
    if constexpr (kPair) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, 2 * BN);
        else tmem_dealloc(tmem_base, 2 * BN);
    }
    if (fuse_own) return;
    // ---------------------------------------------------------------- reduction of this rank's own tiles (more than four ranks)
    const uint64_t* my_flags = reinterpret_cast<const uint64_t*>(c.heap[c.rank] + flag_off);
    const uint8_t* my_part = c.heap[c.rank] + part_off;
    const uint64_t target = static_cast<uint64_t>(p.flag_target);
    for (int lt = bid; lt < tiles_per_dst; lt += nctas) {
        if (threadIdx.x < R) {
            const uint64_t* flag = my_flags + static_cast<uint64_t>(threadIdx.x) * tiles_per_dst + lt;
            if (!bounded_wait(w, kStatusTileFlag, threadIdx.x, lt, [&]() { return ld_acquire_sys_u64(flag) >= target; }))
                atomicExch(p.error, static_cast<int>(kStatusTileFlag));
        }
        __syncthreads();
        const int local_m0 = (lt / tiles_n) * BM, n0 = (lt % tiles_n) * BN;
        // Two 16-byte columns per thread and pass, all sources loaded before the first add: up to 16 loads in flight
        // per thread, so the phase runs at memory speed instead of one load latency per source.
        for (int v0 = threadIdx.x; v0 < BM * BN / 8; v0 += 2 * blockDim.x) {
            int4 raw[2][kMaxRanks];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = v0 + u * blockDim.x;
                const int r = v / (BN / 8), cv = v % (BN / 8);
#pragma unroll
                for (int s = 0; s < kMaxRanks; ++s)
                    if (s < R && v < BM * BN / 8)
                        raw[u][s] = ld_nc_int4(my_part + ((static_cast<uint64_t>(s) * Ml + local_m0 + r) * N + n0 + cv * 8) * 2);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = v0 + u * blockDim.x;
                if (v >= BM * BN / 8) break;
                const int r = v / (BN / 8), cv = v % (BN / 8);
                float accv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) accv[i] = 0.f;
#pragma unroll
                for (int s = 0; s < kMaxRanks; ++s) {
                    if (s < R) {
                        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u][s]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(h2[i]);
                            accv[2 * i] += f.x;
                            accv[2 * i + 1] += f.y;
                        }
                    }
                }
                int4 out;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(accv[2 * i], accv[2 * i + 1]);
                *reinterpret_cast<int4*>(p.out + (static_cast<int64_t>(local_m0 + r) * p.ldo + n0 + cv * 8)) = out;
            }
        }
        __syncthreads();
    }
}

}  // namespace

static bool tp_pairs_enabled() {
    const char* e = std::getenv("EP_TP_CTA_PAIR");
    return e == nullptr || e[0] != '0';
}

// cooperative launch (all CTAs resident: they wait for one another) in clusters of two
template <typename Kernel, typename Launch>
static cudaError_t coop_pairs(Kernel kernel, const Launch& L, int grid, int block, int smem, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, L);
}

static cudaError_t coop(const void* fn, void* arg, int grid, int block, int smem, cudaStream_t stream) {
    void* args[] = {arg};
    return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(block), args, smem, stream);
}

cudaError_t launch_ag_gemm(const AgGemmParams* params, const void* const* b, const void* const* gather_base, int num_vranks,
                           int ctas_per_rank, cudaStream_t stream) {
    if (num_vranks < 1 || num_vranks > kTpMaxVRanks) return cudaErrorInvalidValue;
    AgLaunch L;
    L.num_vranks = num_vranks;
    L.ctas_per_rank = ctas_per_rank;
    // CTA pairs: comm CTAs and GEMM CTAs must both come in twos, and the arrival order must have an even length
    bool pair = tp_pairs_enabled() && ctas_per_rank % 2 == 0;
    for (int v = 0; v < num_vranks; ++v)
        pair = pair && params[v].num_comm_ctas % 2 == 0 && (params[v].c.num_ranks * (params[v].rows_per_rank / BM)) % 2 == 0;
    for (int v = 0; v < num_vranks; ++v) {
        const AgGemmParams& p = params[v];
        const int R = p.c.num_ranks;
        if (p.N % BN != 0 || p.K % BK != 0 || p.rows_per_rank % BM != 0 || p.rows_per_rank / BM > 63) return cudaErrorInvalidValue;
        if (p.num_comm_ctas >= ctas_per_rank) return cudaErrorInvalidValue;
        // the comm warps stage two rows (K * 2 bytes) each
        if (2 * 6 * (align_up(p.K * 2, 128) + 16) > kAgSmem - 1024) return cudaErrorInvalidValue;
        L.p[v] = p;
        if (!make_kmajor_map(&L.map_local[v], p.a_local, 2, p.rows_per_rank, p.K, p.a_stride_bytes, BM) ||
            !make_kmajor_map(&L.map_gather[v], gather_base[v], 2, static_cast<uint64_t>(R) * p.rows_per_rank, p.K, static_cast<uint64_t>(p.K) * 2, BM) ||
            !make_kmajor_map(&L.map_b[v], b[v], 2, p.N, p.K, static_cast<uint64_t>(p.K) * 2, pair ? BN / 2 : BN))
            return cudaErrorInvalidValue;
    }
    if (pair) {
        cudaError_t err = cudaFuncSetAttribute(ag_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AgCfg<true>::kSmem);
        if (err != cudaSuccess) return err;
        return coop_pairs(ag_gemm_kernel<true>, L, num_vranks * ctas_per_rank, kAgThreads, AgCfg<true>::kSmem, stream);
    }
    cudaError_t err = cudaFuncSetAttribute(ag_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAgSmem);
    if (err != cudaSuccess) return err;
    return coop(reinterpret_cast<const void*>(ag_gemm_kernel<false>), &L, num_vranks * ctas_per_rank, kAgThreads, kAgSmem, stream);
}

cudaError_t launch_gemm_rs(const GemmRsParams* params, const void* const* a, const int64_t* a_stride_bytes, const void* const* b,
                           int num_vranks, int ctas_per_rank, cudaStream_t stream) {
    if (num_vranks < 1 || num_vranks > kTpMaxVRanks) return cudaErrorInvalidValue;
    RsLaunch L;
    L.num_vranks = num_vranks;
    L.ctas_per_rank = ctas_per_rank;
    // CTA pairs need an even CTA count per rank and an even number of 128-row chunks (EP_TP_CTA_PAIR=0 turns them off)
    bool pair = tp_pairs_enabled() && ctas_per_rank % 2 == 0;
    for (int v = 0; v < num_vranks; ++v) pair = pair && (params[v].rows_per_rank / BM) % 2 == 0;
    for (int v = 0; v < num_vranks; ++v) {
        const GemmRsParams& p = params[v];
        const int R = p.c.num_ranks;
        if (p.N % BN != 0 || p.K % BK != 0 || p.rows_per_rank % BM != 0) return cudaErrorInvalidValue;
        L.p[v] = p;
        if (!make_kmajor_map(&L.map_a[v], a[v], 2, static_cast<uint64_t>(R) * p.rows_per_rank, p.K, a_stride_bytes[v], BM) ||
            !make_kmajor_map(&L.map_b[v], b[v], 2, p.N, p.K, static_cast<uint64_t>(p.K) * 2, pair ? BN / 2 : BN))
            return cudaErrorInvalidValue;
    }
    if (pair) {
        cudaError_t err = cudaFuncSetAttribute(gemm_rs_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, RsCfg<true>::kSmem);
        if (err != cudaSuccess) return err;
        return coop_pairs(gemm_rs_kernel<true>, L, num_vranks * ctas_per_rank, kRsThreads, RsCfg<true>::kSmem, stream);
    }
    cudaError_t err = cudaFuncSetAttribute(gemm_rs_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, RsCfg<false>::kSmem);
    if (err != cudaSuccess) return err;
    return coop(reinterpret_cast<const void*>(gemm_rs_kernel<false>), &L, num_vranks * ctas_per_rank, kRsThreads, RsCfg<false>::kSmem, stream);
}

}  // namespace gemm
}  // namespace ep
