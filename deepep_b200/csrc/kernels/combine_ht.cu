// High-throughput expert-parallel combine for one NVLink/NVSwitch domain (sm_100a).
//
// Send kernel (cooperative, `num_sms` blocks): every received row goes back to the rank it
// came from, into row [lane][token] of that rank's combine region, where `lane` is the
// sending rank (rank layout: one row per contributing rank, a rank's local experts are
// summed in fp32 before the row leaves) or the top-k slot (top-k layout: one row per
// expert, no intermediate rounding). Destinations are visited round-robin starting at
// rank+1 so that at any moment the ranks of the domain target different receivers.
// The combine region is double-buffered by epoch parity, which is what makes an entry
// barrier unnecessary: a peer can only be two combines ahead after this rank has finished
// reading the half it is about to overwrite.
//
// Reduce: combined_x[t] = sum over lanes in ascending order (fp32) + bias_0 + bias_1, one bf16
// rounding at the end; top-k weights are gathered back. Two ways to run it:
//   * arrival-driven, beside the send kernel (default with peers): for every row that has landed the
//     sender adds one to a counter in the RECEIVER's heap (one counter per sender and per 32
//     consecutive rows of what that sender holds for the receiver). A send warp never fences: three
//     rows late, when wait_group has confirmed a row's remote writes, it drops the row's tag into a
//     shared-memory mailbox, and one extra "accountant" warp per block drains all mailboxes, issues
//     ONE `fence.acq_rel.sys` for everything it drained (a system-scope fence costs microseconds on
//     an SM with peer stores in flight, so it is paid per batch, not per row; without it a relaxed
//     add can overtake the row it announces on NVLink) and then the `red.relaxed.sys` adds, so
//     neither the NVLink round trip nor the accounting stalls a send warp; the reduce kernel is
//     launched as a programmatic dependent of the send kernel -- it becomes resident on the SMs the
//     send kernel leaves free once every send block is running -- and sums a token as soon as the
//     counters of all its rows are full, while later rows are still in flight. The counters of one
//     parity are zeroed by the send kernel of the combine before (no peer can be two combines ahead);
//   * the same reduce kernel after the send kernel (no counters), e.g. when an event gates the reduce.
// With `weighted`, expanded rows are multiplied by their top-k weight: in the sender's fp32
// pre-reduce (rank layout) or in the reduce (top-k layout).
//
// Parity: deep_ep/include/deep_ep/impls/combine.cuh:15-243, impls/combine_utils.cuh:41-170
// and impls/combine_reduce_epilogue.cuh:12-143 of the reference.
#include "api.hpp"
#include "../common/device_utils.cuh"

namespace ep {

namespace {

__device__ __forceinline__ void accumulate_bf16x8(float (&acc)[8], const int4& raw) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h2[i]);
        acc[2 * i] += v.x;
        acc[2 * i + 1] += v.y;
    }
}

__device__ __forceinline__ void accumulate_bf16x8_scaled(float (&acc)[8], const int4& raw, float wt) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h2[i]);
        acc[2 * i] = fmaf(wt, v.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(wt, v.y, acc[2 * i + 1]);
    }
}

// top-k layout, weighted: the weight of the row in lane `row` of token t (its own top-k weight)
__device__ __forceinline__ float row_weight(const CombineEpilogueParams& p, int t, int row) {
    return p.region_w[(static_cast<uint64_t>(row) * p.num_max_tokens + t) * p.num_topk + row];
}

__device__ __forceinline__ int4 pack_bf16x8(const float (&acc)[8]) {
    int4 out;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return out;
}

// NV columns (16 bytes each) per lane and pass, rows taken NR at a time.
template <int NV, int NR>
__device__ __forceinline__ void reduce_columns(const CombineEpilogueParams& p, int t, uint32_t mask, int lane, const uint8_t* b0,
                                               const uint8_t* b1) {
    const int vec_per_row = p.hidden / 8;
    const uint64_t row_bytes = static_cast<uint64_t>(p.hidden) * 2;
    for (int v = lane; v < vec_per_row; v += 32 * NV) {
        float acc[NV][8];
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
        uint32_t todo = mask;
        while (todo) {
            int rows[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                rows[r] = todo ? __ffs(todo) - 1 : -1;
                todo &= todo - 1;       // 0 stays 0
            }
            int4 raw[NR][NV];
            float wt[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                wt[r] = (p.weighted && rows[r] >= 0) ? row_weight(p, t, rows[r]) : 1.f;
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (rows[r] >= 0 && v + 32 * j < vec_per_row)
                        raw[r][j] = ld_nc_int4(p.region_x + (static_cast<uint64_t>(rows[r]) * p.num_max_tokens + t) * row_bytes + (v + 32 * j) * 16);
            }
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (rows[r] >= 0 && v + 32 * j < vec_per_row) {
                        if (p.weighted) accumulate_bf16x8_scaled(acc[j], raw[r][j], wt[r]);
                        else accumulate_bf16x8(acc[j], raw[r][j]);
                    }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (v + 32 * j >= vec_per_row) break;
            if (b0 != nullptr) accumulate_bf16x8(acc[j], ld_nc_int4(b0 + (v + 32 * j) * 16));
            if (b1 != nullptr) accumulate_bf16x8(acc[j], ld_nc_int4(b1 + (v + 32 * j) * 16));
            st_na_int4(p.combined_x + t * row_bytes + (v + 32 * j) * 16, pack_bf16x8(acc[j]));
        }
    }
}

// ==================================================================== reduce of one token (one warp)
// combined_x[t] = sum over the lanes that hold a row for the token, ascending, fp32, + bias_0 + bias_1, one bf16 rounding.
// `e` is the lane's expert (-1 = unused top-k lane), identical on both callers.
__device__ __forceinline__ void reduce_token(const CombineEpilogueParams& p, int t, int e, int lane) {
    const int K = p.num_topk, EL = p.num_local_experts;
    const int vec_per_row = p.hidden / 8;
    const uint64_t row_bytes = static_cast<uint64_t>(p.hidden) * 2;
    const int slot_lane = e < 0 ? -1 : (p.use_rank_layout ? e / EL : lane);
    uint32_t mask = slot_lane >= 0 ? (1u << slot_lane) : 0u;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mask |= __shfl_xor_sync(0xffffffffu, mask, o);
    if (p.combined_topk_weights != nullptr && lane < K) {
        float wv = 0.f;
        if (slot_lane >= 0 && p.region_w != nullptr)
            wv = p.region_w[(static_cast<uint64_t>(slot_lane) * p.num_max_tokens + t) * K + lane];
        p.combined_topk_weights[static_cast<int64_t>(t) * K + lane] = wv;
    }
    const uint8_t* b0 = p.bias0 != nullptr ? p.bias0 + t * row_bytes : nullptr;
    const uint8_t* b1 = p.bias1 != nullptr ? p.bias1 + t * row_bytes : nullptr;
    if (__popc(mask) == 1 && b0 == nullptr && b1 == nullptr && !p.weighted) {
        // a single contribution (e.g. one rank): the sum is a copy; keep four loads in flight per lane
        const uint8_t* src = p.region_x + (static_cast<uint64_t>(__ffs(mask) - 1) * p.num_max_tokens + t) * row_bytes;
        uint8_t* dst = p.combined_x + t * row_bytes;
        for (int v = lane; v < vec_per_row; v += 128) {
            int4 raw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v + 32 * j < vec_per_row) raw[j] = ld_nc_int4(src + (v + 32 * j) * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v + 32 * j < vec_per_row) st_na_int4(dst + (v + 32 * j) * 16, raw[j]);
        }
        return;
    }
    // Eight 16-byte loads are in flight per lane before the first add: eight rows of one column, or (when at most
    // four lanes contribute) four rows of two columns. The adds run in ascending lane order either way.
    if (__popc(mask) <= 4)
        reduce_columns<2, 4>(p, t, mask, lane, b0, b1);
    else
        reduce_columns<1, 8>(p, t, mask, lane, b0, b1);
}

__device__ __forceinline__ int token_expert(const CombineEpilogueParams& p, int t, int lane) {
    if (lane >= p.num_topk) return -1;
    return load_topk_idx(p.topk_idx, p.idx32 != 0, static_cast<int64_t>(t) * p.num_topk + lane, p.num_local_experts * p.num_ranks);
}

__device__ __noinline__ void reduce_token_registers(const CombineEpilogueParams& p, int t, int e, int lane) {
    reduce_token(p, t, e, lane);
}

// ==================================================================== reduce epilogue (local, all SMs)
// Rows are staged through shared memory with bulk copies: a warp owns a ring of kEpiSlots chunk slots of 1 KB and keeps
// floor(kEpiSlots / n) chunks of each of a token's n contributing rows in flight (8 deep for two rows, 2 deep for
// eight: the bytes in flight per SM, which set the bandwidth a reduce SM reaches, do not depend on the routing), then
// every lane sums its two 16-byte pieces of the chunk over the rows in ascending lane order. The chunk size matters: every chunk costs a proxy fence, two
// warp barriers and an mbarrier round, and with 512-byte chunks that fixed cost, not memory, set the pace (147 us
// against 130 us for the EP8-shaped case). Tokens with at most one row, more than kEpiRows rows, or a row size that is
// not a multiple of the chunk take the register path (reduce_token).
constexpr int kEpiSlots = 16, kEpiMaxDepth = 8, kEpiRows = 8, kEpiChunk = 1024, kEpiWarps = 12;
constexpr int kEpiWarpBytes = kEpiSlots * kEpiChunk;
constexpr int kEpiSmem = kEpiWarps * kEpiWarpBytes + kEpiWarps * kEpiMaxDepth * 8;

__global__ void __launch_bounds__(kEpiWarps * 32) combine_epilogue_kernel(const __grid_constant__ Multi<CombineEpilogueParams> m) {
    extern __shared__ __align__(128) uint8_t epi_smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const CombineEpilogueParams& p = m.r[vr];
    const int lane = lane_id(), warp = warp_id();
    const int num_warps = blockDim.x >> 5;
    uint8_t* sbuf = epi_smem + static_cast<size_t>(warp) * kEpiWarpBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kEpiWarps * kEpiWarpBytes) + warp * kEpiMaxDepth;
    if (lane == 0) {
        for (int s = 0; s < kEpiMaxDepth; ++s) mbar_init(bars + s, 1);
        fence_mbar_init();
    }
    __syncwarp();
    uint32_t parity = 0;                    // bit s = phase the next wait on stage s expects
    bool staged_ok = true;                  // a wait that ever ran out sends the rest through the register path
    const int K = p.num_topk, EL = p.num_local_experts;
    const uint64_t row_bytes = static_cast<uint64_t>(p.hidden) * 2;
    const int nchunks = static_cast<int>(row_bytes / kEpiChunk);
    const bool chunkable = row_bytes % kEpiChunk == 0;
    const uint64_t deadline = globaltimer_ns() + 2000000000ull;
    uint64_t* timeline = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(p.local_ws) + kWsTimelineOffsetBytes) + 2 * kTlCombineReduce;
    if (bid == 0 && threadIdx.x == 0) timeline[0] = globaltimer_ns();
    // Flag-driven mode: this kernel runs beside the send kernel (it never waits for it as a whole); the tokens of
    // a warp are visited in ascending order, which is also the order in which their rows arrive.
    const bool flagged = p.arrivals != nullptr;
    const WaitCtx w = make_wait_ctx(p.c);
    bool flags_ok = true;
    // per source rank: first row of this rank's tokens in that rank's receive order, and how many rows it holds for us
    __shared__ int s_base[kMaxRanks], s_held[kMaxRanks];
    if (flagged && threadIdx.x < p.num_ranks) {
        const int src = threadIdx.x, me = p.c.rank;
        int base = 0;
        for (int i = 0; i < me; ++i) base += p.count_matrix[i * p.num_ranks + src];
        s_base[src] = base;
        s_held[src] = p.count_matrix[me * p.num_ranks + src];
    }
    __syncthreads();

    for (int t = bid * num_warps + warp; t < p.num_tokens && flags_ok; t += nb * num_warps) {
        const int e = token_expert(p, t, lane);
        if (flagged) {
            bool ok = true;
            if (e >= 0) {
                const int src = e / EL;
                const int slot = p.dst_slot[static_cast<int64_t>(t) * p.num_ranks + src];
                if (slot >= 0) {
                    // position of the row among the rows that `src` holds for this rank, and how many of them share its counter
                    const int idx = slot - s_base[src];
                    const int g = idx / kCombineFlagRows;
                    const uint32_t want = static_cast<uint32_t>(min(kCombineFlagRows, s_held[src] - g * kCombineFlagRows));
                    const uint32_t* cnt = p.arrivals + static_cast<uint64_t>(src) * p.flag_chunks + g;
                    ok = idx >= 0 && bounded_wait(w, kStatusCombineDone, src, t, [&]() { return ld_acquire_sys_u32(cnt) >= want; });
                }
            }
            flags_ok = __all_sync(0xffffffffu, ok);
            if (!flags_ok) break;
            // (the rows are then read with bulk copies, which fetch from L2, where the senders' completed writes are;
            // a full async-proxy fence per token would serialise the warps of the SM at microseconds apiece)
        }
        const int slot_lane = e < 0 ? -1 : (p.use_rank_layout ? e / EL : lane);
        uint32_t mask = slot_lane >= 0 ? (1u << slot_lane) : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mask |= __shfl_xor_sync(0xffffffffu, mask, o);
        const int n = __popc(mask);
        if (!chunkable || !staged_ok || n < 2 || n > kEpiRows) {
            reduce_token_registers(p, t, e, lane);
            continue;
        }
        if (p.combined_topk_weights != nullptr && lane < K) {
            float wv = 0.f;
            if (slot_lane >= 0 && p.region_w != nullptr)
                wv = p.region_w[(static_cast<uint64_t>(slot_lane) * p.num_max_tokens + t) * K + lane];
            p.combined_topk_weights[static_cast<int64_t>(t) * K + lane] = wv;
        }
        const uint8_t* b0 = p.bias0 != nullptr ? p.bias0 + t * row_bytes : nullptr;
        const uint8_t* b1 = p.bias1 != nullptr ? p.bias1 + t * row_bytes : nullptr;
        // lane r < n loads row r = the r-th contributing lane of the region (ascending)
        const int my_slot = lane < n ? static_cast<int>(__fns(mask, 0, lane + 1)) : 0;
        const float my_wt = (p.weighted && lane < n) ? row_weight(p, t, my_slot) : 1.f;
        const uint8_t* my_src = p.region_x + (static_cast<uint64_t>(my_slot) * p.num_max_tokens + t) * row_bytes;
        uint8_t* dst = p.combined_x + t * row_bytes;
        const int depth = min(kEpiMaxDepth, kEpiSlots / n);      // stage s of this token = slots [s * n, (s + 1) * n)
        for (int c = 0; c < nchunks + depth - 1 && staged_ok; ++c) {
            if (c < nchunks) {
                const int s = c % depth;
                fence_proxy_async_smem();       // this stage was read (generic proxy) one iteration ago
                __syncwarp();
                if (lane == 0) mbar_arrive_expect_tx(bars + s, static_cast<uint32_t>(n) * kEpiChunk);
                __syncwarp();
                if (lane < n) bulk_g2s(sbuf + (s * n + lane) * kEpiChunk, my_src + static_cast<uint64_t>(c) * kEpiChunk, kEpiChunk, bars + s);
            }
            if (c >= depth - 1) {
                const int cc = c - (depth - 1), s = cc % depth;
                uint32_t spins = 0;
                bool ok = true;
                while (!mbar_try_wait(bars + s, (parity >> s) & 1u)) {
                    if ((++spins & 1023u) == 0 && globaltimer_ns() > deadline) { ok = false; break; }
                }
                staged_ok = __all_sync(0xffffffffu, ok);
                if (!staged_ok) break;
                parity ^= 1u << s;
#pragma unroll
                for (int h = 0; h < kEpiChunk / 512; ++h) {
                    float acc[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
                    for (int r = 0; r < kEpiRows; ++r) {
                        const float wt = p.weighted ? __shfl_sync(0xffffffffu, my_wt, r) : 1.f;
                        if (r < n) {
                            const int4 raw = *reinterpret_cast<const int4*>(sbuf + (s * n + r) * kEpiChunk + h * 512 + lane * 16);
                            if (p.weighted) accumulate_bf16x8_scaled(acc, raw, wt);
                            else accumulate_bf16x8(acc, raw);
                        }
                    }
                    const int off = cc * kEpiChunk + h * 512 + lane * 16;
                    if (b0 != nullptr) accumulate_bf16x8(acc, ld_nc_int4(b0 + off));
                    if (b1 != nullptr) accumulate_bf16x8(acc, ld_nc_int4(b1 + off));
                    st_na_int4(dst + off, pack_bf16x8(acc));
                }
            }
        }
        if (!staged_ok) reduce_token_registers(p, t, e, lane);     // redo this token the slow way; later tokens skip the staging
    }
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned long long*>(timeline + 1), static_cast<unsigned long long>(globaltimer_ns()));
}

// kFlags: senders count landed rows in the receivers' heaps (a reduce kernel beside this one consumes the counters).
template <bool kFlags>
__global__ void __launch_bounds__(1024, 1) combine_kernel(const __grid_constant__ Multi<CombineParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const CombineParams& p = m.r[vr];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int num_warps = p.num_send_warps;           // warps that send; with kFlags the block carries one more, the accountant
    const int nb_send = p.num_send_blocks;            // blocks [nb_send, nb) have no send warps at all
    const bool is_sender = warp < num_warps && bid < nb_send;
    const int R = c.num_ranks, K = p.num_topk;
    uint64_t* my_ctl = reinterpret_cast<uint64_t*>(c.heap[c.rank]);
    uint64_t* timeline = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsTimelineOffsetBytes) + 2 * kTlCombine;
    if (bid == 0 && tid == 0) timeline[0] = globaltimer_ns();
    // every block of this grid is running: a reduce kernel launched as programmatic dependent may take the free SMs
    launch_dependents();

    const int stage = align_up(p.row_bytes, 128) + 16;
    uint8_t* buf = smem + static_cast<size_t>(is_sender ? warp : 0) * stage;
    uint64_t* bar = reinterpret_cast<uint64_t*>(buf + align_up(p.row_bytes, 128));
    if (is_sender && lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();

    // ---- arrival accounting: a row counts as landed three rows late, when wait_group has confirmed its remote
    // writes to lane 0 of its send warp; that lane drops the row's tag (destination rank << 24 | 32-row group) into
    // its mailbox and carries on. The accountant warp (the warp after the send warps) drains the mailboxes: the tags
    // reach it through shared memory with release / acquire at block scope, so ONE system-scope fence of the
    // accountant orders every drained row (and the top-k weights stored beside it) before the adds that follow.
    // `pend` holds the tags of the last three rows sent, oldest first.
    constexpr int kMboxDepth = 8;      // a warp's last rows are posted together at the end of the kernel
    __shared__ int s_mbox[32][kMboxDepth];
    __shared__ int s_head[32], s_tail[32];
    __shared__ int s_senders_done;
    if (kFlags) {
        if (tid < 32) s_head[tid] = s_tail[tid] = 0;
        if (tid == 0) s_senders_done = 0;
        __syncthreads();
    }
    const bool is_accountant = kFlags && warp == num_warps && bid < nb_send;
    const uint64_t arrivals_off = p.off_comb_flag + static_cast<uint64_t>(p.epoch & 1) * R * p.flag_chunks * 4;
    auto count_rows = [&](int tag, uint32_t n) {
        uint32_t* cnt = reinterpret_cast<uint32_t*>(c.heap[tag >> 24] + arrivals_off) + static_cast<uint64_t>(c.rank) * p.flag_chunks + (tag & 0xffffff);
        asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(n) : "memory");
    };
    int my_head = 0;
    auto row_landed = [&](int tag) {             // lane 0 of a send warp
        int spins = 0;
        while (my_head - *reinterpret_cast<volatile int*>(&s_tail[warp]) >= kMboxDepth) {
            if (++spins > (1 << 22)) {           // the accountant gave up: count the row here, at full price
                fence_acq_rel_sys();
                count_rows(tag, 1u);
                return;
            }
        }
        *reinterpret_cast<volatile int*>(&s_mbox[warp][my_head & (kMboxDepth - 1)]) = tag;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&s_head[warp]) = ++my_head;
    };
    // (Six rows instead of three were measured at EP8: no change, 834 us either way against 791 us for the send kernel
    // without accounting; neither do fewer fences of the accountant or fewer adds explain the difference.)
    int pend0 = -1, pend1 = -1, pend2 = -1;
    auto row_sent = [&](int d, int idx) {        // after bulk_commit of the row's only store
        if (!kFlags) return;
        bulk_wait<3>();
        if (pend0 >= 0) row_landed(pend0);
        pend0 = pend1;
        pend1 = pend2;
        pend2 = (d << 24) | (idx / kCombineFlagRows);
    };
    auto flush_sent = [&]() {
        if (!kFlags) return;
        bulk_wait_all();
        if (pend0 >= 0) row_landed(pend0);
        if (pend1 >= 0) row_landed(pend1);
        if (pend2 >= 0) row_landed(pend2);
        pend0 = pend1 = pend2 = -1;
    };
    if (kFlags) {
        // zero the counters the NEXT combine will count into (the other parity): no peer starts that combine before
        // it has seen this rank's completion word, which is sent at the end of this kernel
        uint32_t* next = reinterpret_cast<uint32_t*>(c.heap[c.rank] + p.off_comb_flag + static_cast<uint64_t>((p.epoch + 1) & 1) * R * p.flag_chunks * 4);
        for (int i = bid * blockDim.x + tid; i < R * p.flag_chunks; i += nb * blockDim.x) next[i] = 0u;
    }

    // groups of received rows per source rank
    int group_begin = 0, group_size = 0, max_group = 0;
    {
        int prev = 0;
        for (int s = 0; s < R; ++s) {
            const int end = p.psum_rank[s];
            const int size = end - prev;
            max_group = max(max_group, size);
            prev = end;
        }
    }
    const int vec_per_row = p.row_bytes / 16;
    uint32_t parity = 0;
    const int64_t total_steps = static_cast<int64_t>(max_group) * R;
    // rows are handed out dynamically (SMs differ in how fast their peer stores drain)
    unsigned long long* work = reinterpret_cast<unsigned long long*>(c.local_ws + kWsWork);
    int64_t g = is_sender ? static_cast<int64_t>(bid) * num_warps + warp : total_steps;
    if (p.direct_out) {
        // tokens without any valid expert receive no row: their result is zero
        const int all_warps = blockDim.x >> 5;
        for (int t = bid * all_warps + warp; t < p.red.num_tokens; t += nb * all_warps) {
            if (__any_sync(0xffffffffu, token_expert(p.red, t, lane) >= 0)) continue;
            for (int v = lane; v < vec_per_row; v += 32)
                st_na_int4(p.red.combined_x + static_cast<uint64_t>(t) * p.row_bytes + v * 16, make_int4(0, 0, 0, 0));
            if (p.red.combined_topk_weights != nullptr && lane < K) p.red.combined_topk_weights[static_cast<int64_t>(t) * K + lane] = 0.f;
        }
    }
    int64_t next_g = 0;
    bool fatal = false;
    for (; g < total_steps && !fatal; g = next_g) {
        // the next index is requested now and only read at the end of the step (latency hidden)
        long long fetched = 0;
        if (lane == 0) fetched = static_cast<long long>(atomicAdd(work, 1ull)) + static_cast<long long>(nb_send) * num_warps;
        do {
        const int d = (c.rank + 1 + static_cast<int>(g % R)) % R;
        const int idx = static_cast<int>(g / R);
        group_begin = d == 0 ? 0 : p.psum_rank[d - 1];
        group_size = p.psum_rank[d] - group_begin;
        if (idx >= group_size) break;
        const int i = group_begin + idx;
        const int* md = p.recv_src_metadata + static_cast<int64_t>(i) * (K + 2);
        const int src_token = md[0] % p.num_max_tokens;
        const int master_lane = md[1] % K;
        uint8_t* heap = c.heap[d];

        bulk_wait_read_all();
        __syncwarp();
        if (!p.do_expand) {
            // one row per received token: forward it as it is
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, p.row_bytes);
                bulk_g2s(buf, p.x + static_cast<int64_t>(i) * p.x_stride_bytes, p.row_bytes, bar);
            }
            const int slot_lane = p.use_rank_layout ? c.rank : master_lane;
            const uint64_t dst_row = static_cast<uint64_t>(slot_lane) * p.num_max_tokens + src_token;
            uint8_t* dst_ptr = heap + p.off_comb_x + dst_row * p.row_bytes;
            if (p.direct_out) {
                // single rank: the row is the token's only contribution, it goes straight to the result
                dst_ptr = p.red.combined_x + static_cast<uint64_t>(src_token) * p.row_bytes;
                if (p.red.combined_topk_weights != nullptr && lane < K)
                    p.red.combined_topk_weights[static_cast<int64_t>(src_token) * K + lane] =
                        token_expert(p.red, src_token, lane) >= 0 && p.topk_weights != nullptr ? p.topk_weights[static_cast<int64_t>(i) * K + lane] : 0.f;
            } else if (p.topk_weights != nullptr && lane < K) {
                reinterpret_cast<float*>(heap + p.off_comb_w)[dst_row * K + lane] = p.topk_weights[static_cast<int64_t>(i) * K + lane];
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, i);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) { fatal = true; break; }
            if (lane == 0) {
                bulk_s2g(dst_ptr, buf, p.row_bytes);
                bulk_commit();
                row_sent(d, idx);
            }
        } else if (p.use_rank_layout) {
            // expanded input: sum this token's local-expert rows in fp32 (ascending top-k lane), round once, send
            int my_row = lane < K ? md[2 + lane] : -1;
            const uint32_t valid = __ballot_sync(0xffffffffu, my_row >= 0);
            const uint64_t dst_row = static_cast<uint64_t>(c.rank) * p.num_max_tokens + src_token;
            uint8_t* dst_ptr = p.direct_out ? p.red.combined_x + static_cast<uint64_t>(src_token) * p.row_bytes
                                            : heap + p.off_comb_x + dst_row * p.row_bytes;
            for (int v = lane; v < vec_per_row; v += 32) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                uint32_t todo = valid;
                while (todo) {      // four rows in flight per lane, added in ascending top-k lane order
                    int rows[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int k = todo ? __ffs(todo) - 1 : -1;
                        todo &= todo - 1;       // 0 stays 0
                        const int row = __shfl_sync(0xffffffffu, my_row, k < 0 ? 0 : k);
                        rows[r] = k < 0 ? -1 : row;
                    }
                    int4 raw[4];
                    float wt[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        if (rows[r] >= 0) raw[r] = ld_nc_int4(p.x + static_cast<int64_t>(rows[r]) * p.x_stride_bytes + v * 16);
                        wt[r] = (p.weighted && rows[r] >= 0) ? p.topk_weights[rows[r]] : 1.f;
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        if (rows[r] >= 0) {
                            if (p.weighted) accumulate_bf16x8_scaled(acc, raw[r], wt[r]);
                            else accumulate_bf16x8(acc, raw[r]);
                        }
                }
                reinterpret_cast<int4*>(buf)[v] = pack_bf16x8(acc);
            }
            if (p.direct_out) {
                if (p.red.combined_topk_weights != nullptr && lane < K)
                    p.red.combined_topk_weights[static_cast<int64_t>(src_token) * K + lane] =
                        my_row >= 0 && p.topk_weights != nullptr ? p.topk_weights[my_row] : 0.f;
            } else if (p.topk_weights != nullptr && my_row >= 0) {
                reinterpret_cast<float*>(heap + p.off_comb_w)[dst_row * K + lane] = p.topk_weights[my_row];
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                bulk_s2g(dst_ptr, buf, p.row_bytes);
                bulk_commit();
                row_sent(d, idx);
            }
        } else {
            // expanded input, top-k layout: every expert row travels on its own
            const int my_row = lane < K ? md[2 + lane] : -1;
            uint32_t todo = __ballot_sync(0xffffffffu, my_row >= 0);
            if (p.topk_weights != nullptr && my_row >= 0)
                reinterpret_cast<float*>(heap + p.off_comb_w)[(static_cast<uint64_t>(lane) * p.num_max_tokens + src_token) * K + lane] = p.topk_weights[my_row];
            bool failed = false;
            while (todo) {
                const int k = __ffs(todo) - 1;
                todo &= todo - 1;
                const int row = __shfl_sync(0xffffffffu, my_row, k);
                bulk_wait_read_all();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar, p.row_bytes);
                    bulk_g2s(buf, p.x + static_cast<int64_t>(row) * p.x_stride_bytes, p.row_bytes, bar);
                }
                const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, row);
                parity ^= 1;
                if (!__all_sync(0xffffffffu, landed)) { failed = true; break; }
                if (lane == 0) {
                    bulk_s2g(heap + p.off_comb_x + (static_cast<uint64_t>(k) * p.num_max_tokens + src_token) * p.row_bytes, buf, p.row_bytes);
                    bulk_commit();
                }
            }
            if (failed) fatal = true;
            if (lane == 0 && kFlags) {     // several stores per token: settle all of them, then count the token
                flush_sent();
                row_landed((d << 24) | (idx / kCombineFlagRows));
            }
        }
        } while (false);
        next_g = __shfl_sync(0xffffffffu, fetched, 0);
    }

    if (lane == 0) flush_sent();
    if (kFlags && is_sender && lane == 0) {
        __threadfence_block();
        atomicAdd(&s_senders_done, 1);
    }
    if (is_accountant) {
        // lane l serves the mailbox of send warp l; the loop ends when every send warp has left and nothing is queued
        int tail = 0;
        uint32_t idle = 0;
        while (true) {
            const int done = *reinterpret_cast<volatile int*>(&s_senders_done);
            const int head = lane < num_warps ? *reinterpret_cast<volatile int*>(&s_head[lane]) : 0;
            __threadfence_block();
            if (__any_sync(0xffffffffu, head != tail)) {
                fence_acq_rel_sys();
                // Rows that the send warps have in flight at one time mostly belong to the same few 32-row groups (rows
                // are handed out in order): lanes with the same tag add once, with their number, so a sweep sends about
                // one add per destination over NVLink instead of one per row.
#pragma unroll 1
                for (int k = 0; k < kMboxDepth; ++k) {
                    const bool has = tail != head;
                    const int tag = has ? *reinterpret_cast<volatile int*>(&s_mbox[lane][tail & (kMboxDepth - 1)]) : (0x7f000000 | lane);
                    if (!__any_sync(0xffffffffu, has)) break;
                    const uint32_t same = __match_any_sync(0xffffffffu, tag);
                    if (has) {
                        if ((same & lanemask_lt()) == 0) count_rows(tag, static_cast<uint32_t>(__popc(same)));
                        ++tail;
                    }
                }
                if (lane < num_warps) *reinterpret_cast<volatile int*>(&s_tail[lane]) = tail;
                idle = 0;
                // A system-scope fence every few microseconds is enough for the reducer and leaves the SM's memory
                // pipes to the send warps in between (a mailbox holds eight rows, a warp sends a row in about 7 us).
                if (done == 0) __nanosleep(4000);        // (not once the first send warp has left: the end of the kernel waits for us)
            } else if (done >= num_warps) {
                break;
            } else if ((++idle & 1023u) == 0 && globaltimer_ns() > w.deadline_ns) {
                break;                           // the send warps record their own time-outs
            }
        }
    }
    __syncwarp();

    // (no fence here: wait_group confirms the rows to their send warps; the grid barrier's release / acquire at GPU
    // scope and the release store of the completion words at system scope order every store of this grid, the top-k
    // weights written with plain peer stores included, before those words)
    bulk_wait_all();
    grid_barrier(w, c.local_ws + kWsGridBarrier, p.grid_bar_base + nb, 3);
    if (bid == 0 && tid == 0) {   // ready for the next launch (stream order)
        c.local_ws[kWsWork] = 0;
    }
    if (bid == 0 && tid < R) {
        uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[tid]) + kCtlCombineDone + c.rank;
        st_release_sys_u64(remote, pack_epoch(p.epoch, 0));
        const uint64_t* word = my_ctl + kCtlCombineDone + tid;
        bounded_wait(w, kStatusCombineDone, tid, 0, [&]() { return epoch_reached(ld_acquire_sys_u64(word), p.epoch); });
    }
    if (tid == 0) atomicMax(reinterpret_cast<unsigned long long*>(timeline + 1), static_cast<unsigned long long>(globaltimer_ns()));
}

}  // namespace

bool plan_combine(const CombineParams& p, int num_sms, int smem_optin, CombineLaunch* out) {
    const int stage = align_up(p.row_bytes, 128) + 16;
    int warps = smem_optin / stage;
    if (warps > 31) warps = 31;        // the 32nd warp of a block is the accountant of the arrival counters
    if (warps < 1) return false;
    out->num_sms = num_sms;
    out->num_warps = warps;
    out->smem_bytes = warps * stage;
    return true;
}

cudaError_t launch_combine(const Multi<CombineParams>& m, const CombineLaunch& l, cudaStream_t stream) {
    void (*kernel)(const Multi<CombineParams>) = m.r[0].fuse_reduce != 0 ? combine_kernel<true> : combine_kernel<false>;
    cudaError_t err = prepare_kernel(kernel, l.smem_bytes);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m.num_vranks * m.blocks_per_rank);
    cfg.blockDim = dim3((l.num_warps + (m.r[0].fuse_reduce != 0 ? 1 : 0)) * 32);     // + the accountant warp
    cfg.dynamicSmemBytes = l.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    Multi<CombineParams> copy = m;
    for (int v = 0; v < copy.num_vranks; ++v) copy.r[v].num_send_warps = l.num_warps;
    // blocks_per_rank counts the reduce-only blocks too

    return cudaLaunchKernelEx(&cfg, kernel, copy);
}

cudaError_t launch_combine_epilogue(const CombineEpilogueParams* params, int num_vranks, int num_sms, cudaStream_t stream,
                                    bool programmatic) {
    Multi<CombineEpilogueParams> m;
    m.num_vranks = num_vranks;
    m.blocks_per_rank = num_sms;
    for (int v = 0; v < num_vranks; ++v) m.r[v] = params[v];
    cudaError_t err = prepare_kernel(combine_epilogue_kernel, kEpiSmem);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_vranks * num_sms);
    cfg.blockDim = dim3(kEpiWarps * 32);
    cfg.dynamicSmemBytes = kEpiSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, combine_epilogue_kernel, m);
}

}  // namespace ep
