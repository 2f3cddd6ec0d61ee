// High-throughput expert-parallel dispatch for one NVLink/NVSwitch domain (sm_100a).
//
// ONE cooperative kernel per rank does, in order:
//   A0. totals   every block counts what its contiguous chunk of tokens sends to each rank and
//                each expert (histogram, no order)
//   B.  exchange block 0 all-gathers this rank's per-rank and per-expert totals into every
//                peer's control area as epoch-tagged words
//   A1. order    while those words travel, every block works out the destination-rank set per
//                token and the position of each (token, rank) and (token, expert) pair among
//                the block's earlier tokens (token order, so the result is the same on every run)
//   B'. bases    every block waits for the whole matrix of totals and derives, without further
//                communication, the first row of its own tokens in each destination's receive
//                region and in each expert's segment of the expanded (expert-major) layout
//   C. send      one warp per token: bulk-load the row into shared memory, optionally cast it
//                to e4m3 with 1x128 scales, append scales and routing words behind the payload,
//                and bulk-store the whole record -- ONE store per destination rank -- straight
//                to record `slot` of that rank's receive region (peer pointers over NVLink;
//                plain 1-D bulk copies, never multicast)
//   D. finish    wait for the own stores; the last block to get there tells every peer "my rows
//                have landed". Nobody waits for the peers here: that wait opens the epilogue.
//
// Records arrive grouped by source rank in token order, i.e. already in the order of the
// non-expanded output: with zero copy the payload column of the receive region IS recv_x (a
// strided view) and the scale column is recv_sf. The epilogue kernel at the bottom is launched
// with programmatic stream serialization, so its blocks are resident before the dispatch
// kernel has drained; it waits for the peers' completion words, unpacks the routing words and
// moves payload rows only when the caller wants tensors of its own or the expanded layout.
//
// Parity: deep_ep/include/deep_ep/impls/dispatch.cuh:17-409 (notify + dispatch warps, one bulk
// store of hidden + SF + metadata per destination at :371-379, programmatic launch of the
// epilogue at :403) and impls/dispatch_copy_epilogue.cuh:11-323 of the reference; the fused
// cast follows the arithmetic of csrc/kernels/legacy/internode_ll.cu:212-249.
#include "api.hpp"
#include "../common/device_utils.cuh"

namespace ep {

namespace {

constexpr int kCntStride = kMaxRanks + kMaxExperts;   // words per source rank in the count matrix
constexpr int kTotOffset = (kMaxBlocks - 1) * (kMaxRanks + kMaxExperts);   // last row of the per-block scratch: totals

// Per-warp staging buffer: [input row][meta as assembled][mbarrier]. Without the fused cast the
// meta sits right behind the payload, so the buffer front IS the record. With the cast the e4m3
// row overwrites the front of the bf16 row (see quantize_row) and the meta is then copied to
// the end of the e4m3 row.
struct StageLayout {
    int meta_off, bar_off, bytes;
};

__host__ __device__ inline StageLayout stage_layout(int src_row_bytes, int meta_bytes) {
    StageLayout s;
    s.meta_off = src_row_bytes;                       // rows are multiples of 16 bytes
    s.bar_off = align_up(s.meta_off + meta_bytes, 16);
    s.bytes = align_up(s.bar_off + 16, 128);
    return s;
}

__host__ __device__ inline int header_bytes(int num_experts) {
    return align_up((3 * kMaxRanks + 2 * num_experts) * 4, 128);
}

// shared memory the ordering pass (A1) needs for one tile of 32 tokens with a single counting warp
__host__ __device__ inline int order_scratch_min_bytes(int num_experts, int num_topk, int num_ranks) {
    return 2 * (2 * num_experts + kMaxRanks) * 4 + 32 * ((num_topk | 1) + (num_ranks | 1)) * 4;
}

// bf16 row in shared memory -> e4m3 row + one float scale per 128 channels. `out` may alias
// `src`: a step covers channels [base, base + 1024), reads bytes [2*base, 2*base + 2048) and
// writes bytes [base, base + 1024), which only earlier steps have read, and the lanes of a step
// have all loaded (the shuffles of the reduction are past) before any of them stores.
// `scales` must not overlap the row.
__device__ __forceinline__ void quantize_row(const uint8_t* src, uint8_t* out, float* scales, int hidden, bool pow2, int lane) {
    constexpr int kUnroll = 4;   // independent 256-channel steps in flight per lane (hides shuffle / divide latency)
    for (int base = 0; base < hidden; base += 256 * kUnroll) {
        int4 raw[kUnroll];
        float amax[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int ch = base + u * 256 + lane * 8;
            raw[u] = ch < hidden ? *reinterpret_cast<const int4*>(src + ch * 2) : make_int4(0, 0, 0, 0);
            amax[u] = amax_bf16x8(raw[u]);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) amax[u] = fmaxf(amax[u], __shfl_xor_sync(0xffffffffu, amax[u], o));
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int ch = base + u * 256 + lane * 8;
            float scale, inv;
            fp8_scale_from_amax(amax[u], pow2, scale, inv);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
            const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
            const float2 c = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
            uint2 packed;
            packed.x = pack4_e4m3(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
            packed.y = pack4_e4m3(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
            if (ch < hidden) {
                *reinterpret_cast<uint2*>(out + ch) = packed;
                if ((lane & 15) == 0) scales[ch >> 7] = scale;
            }
        }
    }
}

__global__ void __launch_bounds__(1024, 1) dispatch_kernel(const __grid_constant__ Multi<DispatchParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_last;
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const DispatchParams& p = m.r[vr];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int tid = threadIdx.x, nthreads = blockDim.x, lane = lane_id(), warp = warp_id();
    const int num_warps = nthreads >> 5;
    const int R = c.num_ranks, E = p.num_experts, K = p.num_topk, T = p.num_tokens, EL = p.num_local_experts;
    const int CW = R + E;
    const bool idx32 = p.idx32 != 0;

    int* s_rank_base = reinterpret_cast<int*>(smem);   // [kMaxRanks] first row of this block's tokens per destination
    int* s_recv_from = s_rank_base + kMaxRanks;         // [kMaxRanks] tokens this rank receives per source
    int* s_flags = s_recv_from + kMaxRanks;             // [kMaxRanks] scratch
    int* s_exp_tot = s_flags + kMaxRanks;               // [E]
    int* s_exp_base = s_exp_tot + E;                    // [E]
    uint8_t* s_bufs = smem + header_bytes(E);

    const int chunk = ceil_div(T, nb);
    const int t0 = min(T, bid * chunk), t1 = min(T, t0 + chunk);
    int* blk_cnt = reinterpret_cast<int*>(c.local_ws + kWsScratch);   // [nb][CW]
    uint64_t* my_ctl = reinterpret_cast<uint64_t*>(c.heap[c.rank]);
    uint64_t* grid_counter = c.local_ws + kWsGridBarrier;
    int* steal_next = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsStealOffsetBytes);   // [nb]
    uint32_t* steal_ready = reinterpret_cast<uint32_t*>(steal_next + kMaxBlocks);                               // [nb]
    int* steal_base = reinterpret_cast<int*>(steal_ready + kMaxBlocks);                                          // [nb][CW]
    uint64_t* timeline = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsTimelineOffsetBytes) + 2 * kTlDispatch;
    bool ok = true;
    // phase timestamps of block 0 (ns, %globaltimer), see kWsStamps
    uint64_t* stamps = c.local_ws + kWsStamps;
    const bool stamper = bid == 0 && tid == 0;
    if (stamper) {
        const uint64_t now = globaltimer_ns();
        stamps[0] = now;
        timeline[0] = now;
    }

    if (!p.cached) {
        // ------------------------------------------------------------ A0. count
        // Totals only: how many tokens this block sends to every rank and how many (token, expert) pairs to
        // every expert. They are all the exchange needs, so they go out first; the order-preserving pass that gives
        // every token its position (A1 below) then runs while the peers' totals are on their way.
        for (int e = tid; e < E; e += nthreads) s_exp_tot[e] = 0;
        if (tid < kMaxRanks) s_flags[tid] = 0;
        __syncthreads();
        for (int base = t0 + warp * 32; base < t1; base += nthreads) {      // a warp takes 32 consecutive tokens
            const int t = base + lane;
            uint32_t mask = 0;
            if (t < t1) {
                for (int k = 0; k < K; ++k) {
                    const int e = load_topk_idx(p.topk_idx, idx32, static_cast<int64_t>(t) * K + k, E);
                    if (e >= 0) {
                        atomicAdd(s_exp_tot + e, 1);
                        mask |= 1u << (e / EL);
                    }
                }
            }
            // one shared-memory atomic per warp and destination rank instead of one per token
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d) {
                if (d < R) {
                    const int n = __popc(__ballot_sync(0xffffffffu, (mask >> d) & 1u));
                    if (lane == d && n != 0) atomicAdd(s_flags + d, n);
                }
            }
        }
        __syncthreads();
        int* tot_cnt = blk_cnt + kTotOffset;   // [CW] totals over the blocks
        for (int j = tid; j < CW; j += nthreads) {
            const int v = j < R ? s_flags[j] : s_exp_tot[j - R];
            blk_cnt[bid * CW + j] = v;
            if (v != 0) atomicAdd(tot_cnt + j, v);
        }
        // (the barrier's block-wide sync followed by its release at GPU scope publishes the counts above)
        ok &= grid_barrier(w, grid_counter, p.grid_bar_base + nb, 1);
        if (stamper) stamps[1] = globaltimer_ns();

        // ------------------------------------------------------------ B. exchange (send the totals, sum the earlier blocks)
        for (int j = tid; j < CW; j += nthreads) {
            if (bid == 0) {
                const uint64_t word = pack_epoch(p.epoch, static_cast<uint32_t>(__ldcg(tot_cnt + j)));
                const int col = j < R ? j : kMaxRanks + (j - R);
                for (int d = 0; d < R; ++d) {
                    uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[d]) + kCtlDispatchCnt + static_cast<size_t>(c.rank) * kCntStride + col;
                    st_relaxed_sys_u64(remote, word);
                }
            }
            // counts of the earlier blocks: 32 independent loads in flight per round
            int before = 0;
            for (int b0 = 0; b0 < bid; b0 += 32) {
                int v[32];
#pragma unroll
                for (int u = 0; u < 32; ++u) v[u] = (b0 + u < bid) ? __ldcg(blk_cnt + (b0 + u) * CW + j) : 0;
#pragma unroll
                for (int u = 0; u < 32; ++u) before += v[u];
            }
            if (j < R) s_rank_base[j] = before; else s_exp_base[j - R] = before;
        }
        // ------------------------------------------------------------ A1. positions of this block's tokens
        // The routing of the chunk is staged in shared memory (the send buffers are idle now).
        // The chunk is cut into contiguous sub-ranges, one per counting warp; every warp ranks its
        // (token, rank) and (token, expert) pairs among its own earlier tokens, a prefix over the
        // warps turns that into positions inside the block. Everything is in token order, so the
        // result does not depend on timing.
        const int scratch_bytes = p.smem_scratch_bytes;
        int cw = num_warps;
        const int per_warp = (2 * E + kMaxRanks) * 4;
        // a lane works on one token: odd row pitches keep the lanes' words of a column in different banks
        const int Kp = K | 1, Rp = R | 1;
        while (cw > 1 && (cw * per_warp > scratch_bytes / 2 || scratch_bytes - cw * per_warp < 32 * (Kp + Rp) * 4)) --cw;
        int* s_wcnt = reinterpret_cast<int*>(s_bufs);          // [cw][E]  per-warp expert counters, then bases
        uint32_t* s_wmask = reinterpret_cast<uint32_t*>(s_wcnt + cw * E);   // [cw][E]  which tokens of the warp's current batch of 32 chose an expert
        int* s_wrank = reinterpret_cast<int*>(s_wmask + cw * E);            // [cw][kMaxRanks]
        int* s_idx = s_wrank + cw * kMaxRanks;                  // [cap_tokens][Kp]
        // (the launcher guarantees room for at least one tile of 32 tokens)
        const int cap_tokens = max(32, ((scratch_bytes - cw * per_warp) / ((Kp + Rp) * 4)) & ~31);
        int* s_slot = s_idx + cap_tokens * Kp;                  // [cap_tokens][Rp]
        __syncthreads();
        for (int e = tid; e < E; e += nthreads) s_exp_tot[e] = 0;
        if (tid < kMaxRanks) s_flags[tid] = 0;
        for (int tile0 = t0; tile0 < t1; tile0 += cap_tokens) {
            const int tile1 = min(t1, tile0 + cap_tokens);
            const int n_tok = tile1 - tile0;
            const int n_pairs = n_tok * K;
            const int tpw = ceil_div(n_tok, cw);
            __syncthreads();
            for (int i = tid; i < n_pairs; i += nthreads)
                s_idx[(i / K) * Kp + i % K] = load_topk_idx(p.topk_idx, idx32, static_cast<int64_t>(tile0) * K + i, E);
            for (int i = tid; i < 2 * cw * E; i += nthreads) s_wcnt[i] = 0;      // counters and masks
            __syncthreads();
            if (warp < cw) {
                const int a = min(n_tok, warp * tpw), b = min(n_tok, a + tpw);
                int run[kMaxRanks];
#pragma unroll
                for (int d = 0; d < kMaxRanks; ++d) run[d] = 0;
                for (int base = a; base < b; base += 32) {
                    const int t = base + lane;
                    uint32_t mask = 0;
                    if (t < b) {
                        for (int k = 0; k < K; ++k) {
                            const int e = s_idx[t * Kp + k];
                            if (e >= 0) mask |= 1u << (e / EL);
                        }
                    }
#pragma unroll
                    for (int d = 0; d < kMaxRanks; ++d) {
                        if (d < R) {
                            const bool in = (mask >> d) & 1u;
                            const uint32_t bal = __ballot_sync(0xffffffffu, in);
                            if (t < b) s_slot[t * Rp + d] = in ? run[d] + __popc(bal & lanemask_lt()) : -1;
                            run[d] += __popc(bal);
                        }
                    }
                }
#pragma unroll
                for (int d = 0; d < kMaxRanks; ++d)
                    if (lane == d) s_wrank[warp * kMaxRanks + d] = run[d];
                // (token, expert) pairs, 32 tokens at a time, one token per lane: every lane marks its experts in a
                // per-expert bit mask; a pair's position is the warp's running count of the expert plus the number of
                // lower lanes in the mask; the lowest lane of a mask then adds the batch to the count and clears the
                // mask. (A warp-wide match on the expert id does the same in one instruction per 32 pairs, but that
                // instruction was measured at about 0.7 us: 5 us for 340 tokens per block.) Experts are assumed
                // distinct within a token, as in the reference.
                int* mine = s_wcnt + warp * E;
                uint32_t* mask_of = s_wmask + warp * E;
                for (int base = a; base < b; base += 32) {
                    const int t = base + lane;
                    if (t < b) {
                        for (int k = 0; k < K; ++k) {
                            const int e = s_idx[t * Kp + k];
                            if (e >= 0) atomicOr(mask_of + e, 1u << lane);
                        }
                    }
                    __syncwarp();
                    if (t < b) {
                        for (int k = 0; k < K; ++k) {
                            const int e = s_idx[t * Kp + k];
                            if (e >= 0) s_idx[t * Kp + k] = ((mine[e] + __popc(mask_of[e] & lanemask_lt())) << 11) | e;
                        }
                    }
                    __syncwarp();
                    if (t < b) {
                        for (int k = 0; k < K; ++k) {
                            const int packed = s_idx[t * Kp + k];
                            if (packed < 0) continue;
                            const int e = packed & 2047;
                            const uint32_t m = mask_of[e];
                            if (m != 0 && (m & lanemask_lt()) == 0) {
                                mine[e] += __popc(m);
                                mask_of[e] = 0;
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            __syncthreads();
            for (int e = tid; e < E; e += nthreads) {
                int acc = s_exp_tot[e];
                for (int wi = 0; wi < cw; ++wi) {
                    const int v = s_wcnt[wi * E + e];
                    s_wcnt[wi * E + e] = acc;
                    acc += v;
                }
                s_exp_tot[e] = acc;
            }
            if (tid < R) {
                int acc = s_flags[tid];
                for (int wi = 0; wi < cw; ++wi) {
                    const int v = s_wrank[wi * kMaxRanks + tid];
                    s_wrank[wi * kMaxRanks + tid] = acc;
                    acc += v;
                }
                s_flags[tid] = acc;
            }
            __syncthreads();
            for (int i = tid; i < n_pairs; i += nthreads) {
                const int packed = s_idx[(i / K) * Kp + i % K];
                const int wi = (i / K) / tpw;
                p.pair_row[static_cast<int64_t>(tile0) * K + i] = packed < 0 ? -1 : s_wcnt[wi * E + (packed & 2047)] + (packed >> 11);
            }
            for (int i = tid; i < n_tok * R; i += nthreads) {
                const int v = s_slot[(i / R) * Rp + i % R];
                const int wi = (i / R) / tpw;
                p.token_slot[static_cast<int64_t>(tile0) * R + i] = v < 0 ? -1 : v + s_wrank[wi * kMaxRanks + (i % R)];
            }
        }
        __syncthreads();
        if (stamper) stamps[2] = globaltimer_ns();
        // ------------------------------------------------------------ B'. the peers' totals -> first rows
        for (int j = tid; j < CW; j += nthreads) {
            const int col = j < R ? j : kMaxRanks + (j - R);
            const uint64_t* words = my_ctl + kCtlDispatchCnt + col;
            uint64_t v[kMaxRanks];
            ok &= bounded_wait(w, kStatusDispatchCounts, -1, j, [&]() {
                bool all = true;
#pragma unroll
                for (int s = 0; s < kMaxRanks; ++s) {
                    if (s < R) {
                        v[s] = ld_relaxed_sys_u64(words + static_cast<size_t>(s) * kCntStride);
                        all &= epoch_matches(v[s], p.epoch);
                    }
                }
                return all;
            });
            int tot = 0, pre = 0;
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) {
                if (s < R) {
                    const int cnt = static_cast<int>(static_cast<uint32_t>(v[s]));
                    tot += cnt;
                    if (s < c.rank) pre += cnt;
                    if (j == c.rank) s_recv_from[s] = cnt;
                    if (j < R && bid == 0 && p.count_matrix != nullptr) p.count_matrix[s * R + j] = cnt;
                }
            }
            if (j < R) {
                s_rank_base[j] += pre;
            } else {
                s_exp_tot[j - R] = tot;
                s_exp_base[j - R] += pre;
            }
        }
        ok = !__syncthreads_or(!ok);
        if (stamper) stamps[3] = globaltimer_ns();
        if (ok) {
            // First row of every expert's segment on its rank (alignment applied): one warp per
            // destination rank runs an exclusive scan over that rank's experts. The warp that scans
            // this rank's own experts in block 0 also writes the receive-side description.
            for (int d = warp; d < R; d += num_warps) {
                const bool owner = bid == 0 && d == c.rank;
                int carry = 0;
                for (int base = 0; base < EL; base += 32) {
                    const int le = base + lane;
                    const int e = d * EL + le;
                    const int tot = le < EL ? s_exp_tot[e] : 0;
                    const int aligned = align_up(tot, p.expert_alignment);
                    int incl = aligned;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int up = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += up;
                    }
                    const int start = carry + incl - aligned;
                    if (le < EL) {
                        s_exp_base[e] += start;
                        if (owner) {
                            p.num_unaligned[le] = tot;
                            p.psum_expert[le] = p.do_expand ? start + tot : start + aligned;
                            if (p.recv_stats != nullptr) p.recv_stats[le] += tot;
                            if (p.host_counts != nullptr) p.host_counts[2 + le] = pack_epoch(p.epoch, static_cast<uint32_t>(aligned));
                        }
                    }
                    carry += __shfl_sync(0xffffffffu, incl, 31);
                }
                if (owner && lane == 0) {
                    p.psum_expert[EL] = carry;
                    if (p.host_counts != nullptr) p.host_counts[1] = pack_epoch(p.epoch, static_cast<uint32_t>(carry));
                }
            }
            if (bid == 0 && warp == num_warps - 1) {
                int incl = lane < R ? s_recv_from[lane] : 0;
#pragma unroll
                for (int o = 1; o < kMaxRanks; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                if (lane < R) p.psum_rank[lane] = incl;
                if (lane == R - 1 && p.host_counts != nullptr) p.host_counts[0] = pack_epoch(p.epoch, static_cast<uint32_t>(incl));
            }
        }
        __syncthreads();
        // Publish the first rows of this block's chunk: a block that runs out of own tokens takes tokens of
        // other chunks and needs their bases (no grid barrier, only a per-block "published" word).
        if (ok) {
            for (int j = tid; j < CW; j += nthreads) steal_base[bid * CW + j] = j < R ? s_rank_base[j] : s_exp_base[j - R];
        }
        __syncthreads();    // ... and the release below (GPU scope, cumulative) publishes what the block wrote
        if (tid == 0 && ok) st_release_gpu_u32(steal_ready + bid, p.epoch);
    } else {
        // ------------------------------------------------------------ cached: only announce entry and wait for the peers
        if (bid == 0 && tid < R) {
            uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[tid]) + kCtlDispatchEntry + c.rank;
            st_release_sys_u64(remote, pack_epoch(p.epoch, 0));
        }
        if (tid < R) {
            const uint64_t* word = my_ctl + kCtlDispatchEntry + tid;
            ok &= bounded_wait(w, kStatusEntry, tid, 0, [&]() { return epoch_reached(ld_acquire_sys_u64(word), p.epoch); });
        }
        ok = !__syncthreads_or(!ok);
    }

    if (stamper) stamps[4] = globaltimer_ns();
    // ---------------------------------------------------------------- C. send
    const bool quant = p.quant_mode != kQuantNone;
    const StageLayout sl = stage_layout(p.src_row_bytes, p.meta_bytes);
    uint8_t* buf = s_bufs + static_cast<size_t>(warp) * sl.bytes;      // input row; its front becomes the record
    uint8_t* buf_meta = buf + sl.meta_off;                              // meta as assembled
    uint8_t* rec_meta = buf + p.x_row_bytes;                            // meta inside the record (== buf_meta without the cast)
    uint64_t* bar = reinterpret_cast<uint64_t*>(buf + sl.bar_off);
    const int rec_bytes = p.x_row_bytes + p.meta_bytes;
    if (ok) {
        if (lane == 0) {
            mbar_init(bar, 1);
            fence_mbar_init();
        }
        __syncwarp();
        const bool sf_in = p.sf != nullptr && p.sf_bytes > 0;
        const bool sf_bulk = sf_in && p.sf_pack_stride == 1 && (p.sf_bytes & 15) == 0 &&
                             ((reinterpret_cast<uintptr_t>(p.sf) | static_cast<uintptr_t>(p.sf_token_stride * 4)) & 15) == 0;
        int* meta_idx = reinterpret_cast<int*>(buf_meta + p.sf_bytes);
        float* meta_w = reinterpret_cast<float*>(meta_idx + K);
        int* meta_row = meta_idx + 2 * K;
        uint32_t parity = 0;
        // Tokens are handed out dynamically: SMs differ in how fast their peer stores drain, and a static
        // split would leave the fast ones idle. Every chunk has a counter; a block serves its own chunk
        // first and then walks the other chunks, taking whatever tokens are left there.
        int victim = bid, v_t0 = t0, v_t1 = t1;
        int t_local = 0;
        if (lane == 0) t_local = atomicAdd(steal_next + victim, 1);
        t_local = __shfl_sync(0xffffffffu, t_local, 0);
        while (true) {
            bool victim_ok = true;
            while (v_t0 + t_local >= v_t1) {
                // Own chunk (or the current victim) is exhausted: look at the counters of the next chunks,
                // 32 at a time, and take a token from the first one that still has some.
                int found = -1;
                for (int off = 1; off < nb && found < 0; off += 32) {
                    const int cand = (bid + off + lane) % nb;
                    bool has = false;
                    if (off + lane < nb) {
                        const int c0 = min(T, cand * chunk), c1 = min(T, c0 + chunk);
                        has = c0 + __ldcg(steal_next + cand) < c1;
                    }
                    const uint32_t bal = __ballot_sync(0xffffffffu, has);
                    if (bal != 0) found = (bid + off + (__ffs(bal) - 1)) % nb;
                }
                if (found < 0) { victim = -1; break; }
                victim = found;
                v_t0 = min(T, victim * chunk);
                v_t1 = min(T, v_t0 + chunk);
                if (lane == 0) t_local = atomicAdd(steal_next + victim, 1);
                t_local = __shfl_sync(0xffffffffu, t_local, 0);
                if (!p.cached && v_t0 + t_local < v_t1) {
                    // the victim's bases must be published (they are, unless it is still in its prologue)
                    victim_ok = bounded_wait(w, kStatusGridBarrier, victim, 5, [&]() { return ld_acquire_gpu_u32(steal_ready + victim) == p.epoch; });
                    victim_ok = __all_sync(0xffffffffu, victim_ok);
                    if (!victim_ok) break;
                }
            }
            if (victim < 0 || !victim_ok) break;
            const int t = v_t0 + t_local;
            const bool foreign = victim != bid;
            int fetched = 0;
            if (lane == 0) fetched = atomicAdd(steal_next + victim, 1);   // next index, read at the end of the step
            bulk_wait_read_all();   // the previous stores of every lane have read the buffer
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, p.src_row_bytes + (sf_bulk ? p.sf_bytes : 0));
                bulk_g2s(buf, p.x + static_cast<int64_t>(t) * p.x_stride_bytes, p.src_row_bytes, bar);
                if (sf_bulk) bulk_g2s(buf_meta, p.sf + static_cast<int64_t>(t) * p.sf_token_stride * 4, p.sf_bytes, bar);
            }
            int slot = -1;
            if (lane < R) {
                slot = p.token_slot[static_cast<int64_t>(t) * R + lane];
                if (!p.cached && slot >= 0) {   // block-relative -> absolute, kept in the handle for cached replays and the combine
                    slot += foreign ? __ldcg(steal_base + victim * CW + lane) : s_rank_base[lane];
                    p.token_slot[static_cast<int64_t>(t) * R + lane] = slot;
                }
            }
            if (lane < K) {
                const int64_t pi = static_cast<int64_t>(t) * K + lane;
                const int e = load_topk_idx(p.topk_idx, idx32, pi, E);
                int row = p.pair_row[pi];
                if (!p.cached && e >= 0) {
                    row += foreign ? __ldcg(steal_base + victim * CW + R + e) : s_exp_base[e];
                    p.pair_row[pi] = row;
                }
                meta_idx[lane] = e;
                meta_w[lane] = p.topk_weights != nullptr ? p.topk_weights[pi] : 0.f;
                meta_row[lane] = row;
            }
            if (lane == 0) meta_row[K] = t;
            if (sf_in && !sf_bulk) {
                const uint32_t* sf32 = reinterpret_cast<const uint32_t*>(p.sf);
                for (int i = lane; i < p.sf_bytes / 4; i += 32)
                    reinterpret_cast<uint32_t*>(buf_meta)[i] = sf32[static_cast<int64_t>(t) * p.sf_token_stride + i * p.sf_pack_stride];
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, t);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) break;
            if (quant) {
                quantize_row(buf, buf, reinterpret_cast<float*>(buf_meta), p.src_row_bytes / 2, p.quant_mode == kQuantE4M3Pow2, lane);
                __syncwarp();       // every lane is done with the bf16 row: its tail may now take the meta
                for (int i = lane; i < p.meta_bytes / 16; i += 32)
                    reinterpret_cast<int4*>(rec_meta)[i] = reinterpret_cast<const int4*>(buf_meta)[i];
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (slot >= 0) {
                bulk_s2g(c.heap[lane] + p.off_recv + static_cast<uint64_t>(slot) * p.rec_pitch, buf, rec_bytes);
                bulk_commit();
            }
            t_local = __shfl_sync(0xffffffffu, fetched, 0);
        }
    }

    // ---------------------------------------------------------------- D. finish
    if (stamper) stamps[5] = globaltimer_ns();
    launch_dependents();          // the epilogue's blocks may become resident from here on
    // wait_group confirms that the records have been written. No fence follows: fences at system scope and full
    // async-proxy fences were measured at 5 to 7 us each while stores of other warps are still in flight, and the chain
    // below (block-wide barrier, acquire-release add on the grid counter, release store of the completion words by the
    // last block) already orders every store of this grid before the completion words.
    bulk_wait_all();
    if (stamper) stamps[6] = globaltimer_ns();
    // The last block to arrive cleans up and tells the peers; nobody spins here.
    __syncthreads();
    if (tid == 0) {
        const uint64_t target = p.grid_bar_base + (p.cached ? 1 : 2) * static_cast<uint64_t>(nb);
        s_last = atom_add_acq_rel_gpu_u64(grid_counter, 1) + 1 == target;
    }
    __syncthreads();
    if (!s_last) return;
    for (int b = tid; b < nb; b += nthreads) steal_next[b] = 0;      // ready for the next launch (stream order)
    if (!p.cached) {
        int* tot_cnt = blk_cnt + kTotOffset;
        for (int j = tid; j < CW; j += nthreads) tot_cnt[j] = 0;
    }
    if (tid < R) {
        uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[tid]) + kCtlDispatchDone + c.rank;
        st_release_sys_u64(remote, pack_epoch(p.epoch, 0));
    }
    if (tid == 0) {
        const uint64_t now = globaltimer_ns();
        stamps[7] = now;
        timeline[1] = now;
    }
}

// ==================================================================== epilogue (local, all SMs)
// 1. waits (bounded) until every peer has reported the rows of this dispatch as landed;
// 2. routing words of all records -> recv_topk_idx (local expert ids), recv_topk_weights, recv_src_metadata,
//    one thread per (record, top-k lane); scale factors -> recv_sf unless the caller reads them in place;
// 3. payload rows -> recv_x[i] (own tensor) or to every expanded row of the token, one warp per record
//    through shared memory (1-D bulk copies); skipped entirely for zero copy;
// 4. zeroes the alignment gaps of the expanded layout when asked to.
__global__ void __launch_bounds__(1024, 1) dispatch_epilogue_kernel(const __grid_constant__ Multi<DispatchEpilogueParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const DispatchEpilogueParams& p = m.r[vr];
    const int tid = threadIdx.x, nthreads = blockDim.x, lane = lane_id(), warp = warp_id();
    const int num_warps = nthreads >> 5;
    const int R = p.num_ranks, K = p.num_topk, EL = p.num_local_experts;
    const bool move_rows = p.copy_x || p.do_expand;
    uint64_t* timeline = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(p.c.local_ws) + kWsTimelineOffsetBytes) + 2 * kTlDispatchEpilogue;

    const int stage = align_up(p.x_row_bytes, 128) + 16;
    uint8_t* buf = smem + static_cast<size_t>(warp) * stage;
    uint64_t* bar = reinterpret_cast<uint64_t*>(buf + align_up(p.x_row_bytes, 128));
    if (move_rows && lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();

    dependency_wait();      // the dispatch kernel of this rank has completed (all its writes are visible)
    if (bid == 0 && tid == 0) timeline[0] = globaltimer_ns();
    const WaitCtx w = make_wait_ctx(p.c);
    bool ok = true;
    if (p.wait_done && tid < R) {
        const uint64_t* word = reinterpret_cast<const uint64_t*>(p.c.heap[p.c.rank]) + kCtlDispatchDone + tid;
        ok = bounded_wait(w, kStatusDispatchDone, tid, 0, [&]() { return epoch_reached(ld_acquire_sys_u64(word), p.epoch); });
    }
    ok = !__syncthreads_or(!ok);
    if (!ok) return;        // the status word says why; the outputs stay as they are

    const int N = min(p.psum_rank[R - 1], p.num_idx_rows);
    const int expert_begin = p.c.rank * EL;
    const int sf_packs = p.sf_bytes / 4;
    const int64_t gtid = static_cast<int64_t>(bid) * nthreads + tid, gthreads = static_cast<int64_t>(nb) * nthreads;
    const bool idx32 = p.idx32 != 0;
    auto meta_of = [&](int i) { return reinterpret_cast<const int*>(p.region + static_cast<uint64_t>(i) * p.rec_pitch + p.x_row_bytes + p.sf_bytes); };

    // ---- 2. routing words, one thread per (record, lane); rows past the received count get -1 / 0
    for (int64_t j = gtid; j < static_cast<int64_t>(p.num_idx_rows) * K; j += gthreads) {
        const int i = static_cast<int>(j / K), k = static_cast<int>(j % K);
        int local_e = -1, row = -1;
        float wt = 0.f;
        if (i < N) {
            const int* mi = meta_of(i);
            const int e = mi[k];
            wt = reinterpret_cast<const float*>(mi)[K + k];
            const bool local = e >= expert_begin && e < expert_begin + EL;
            local_e = local ? e - expert_begin : -1;
            if (p.do_expand && local) row = mi[2 * K + k];
            if (row >= p.num_out_rows) row = -1;
            if (p.write_metadata && k == 0) {
                int first_local = 0;
                for (int kk = K - 1; kk >= 0; --kk) {
                    const int ee = mi[kk];
                    if (ee >= expert_begin && ee < expert_begin + EL) first_local = kk;
                }
                int src_rank = 0;
                for (int r = 0; r < R - 1; ++r) src_rank += i >= p.psum_rank[r];
                int* md = p.recv_src_metadata + static_cast<int64_t>(i) * (K + 2);
                md[0] = src_rank * p.num_max_tokens + mi[3 * K];
                md[1] = src_rank * K + first_local;
            }
        } else if (p.write_metadata && k == 0) {
            int* md = p.recv_src_metadata + static_cast<int64_t>(i) * (K + 2);
            md[0] = -1;
            md[1] = -1;
        }
        if (!p.do_expand) {
            if (p.recv_topk_idx != nullptr) {
                if (idx32) reinterpret_cast<int*>(p.recv_topk_idx)[j] = local_e;
                else reinterpret_cast<int64_t*>(p.recv_topk_idx)[j] = local_e;
            }
            if (p.recv_topk_weights != nullptr) p.recv_topk_weights[j] = wt;
        } else if (row >= 0 && p.recv_topk_weights != nullptr) {
            p.recv_topk_weights[row] = wt;
        }
        if (p.write_metadata) p.recv_src_metadata[static_cast<int64_t>(i) * (K + 2) + 2 + k] = row;
    }

    // ---- scale factors, one thread per (record, pack)
    if (p.recv_sf != nullptr && sf_packs > 0) {
        uint32_t* out = reinterpret_cast<uint32_t*>(p.recv_sf);
        for (int64_t j = gtid; j < static_cast<int64_t>(N) * sf_packs; j += gthreads) {
            const int i = static_cast<int>(j / sf_packs), k = static_cast<int>(j % sf_packs);
            const uint32_t v = reinterpret_cast<const uint32_t*>(p.region + static_cast<uint64_t>(i) * p.rec_pitch + p.x_row_bytes)[k];
            if (!p.do_expand) {
                if (i < p.num_out_rows) out[static_cast<int64_t>(i) * p.recv_sf_row_stride + static_cast<int64_t>(k) * p.recv_sf_pack_stride] = v;
            } else {
                const int* mi = meta_of(i);
                for (int kk = 0; kk < K; ++kk) {
                    const int e = mi[kk];
                    if (e < expert_begin || e >= expert_begin + EL) continue;
                    const int row = mi[2 * K + kk];
                    if (row >= 0 && row < p.num_out_rows)
                        out[static_cast<int64_t>(row) * p.recv_sf_row_stride + static_cast<int64_t>(k) * p.recv_sf_pack_stride] = v;
                }
            }
        }
    }

    // ---- 3. payload rows, one warp per record
    if (move_rows) {
        uint32_t parity = 0;
        for (int i = bid * num_warps + warp; i < N; i += nb * num_warps) {
            bulk_wait_read_all();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, p.x_row_bytes);
                bulk_g2s(buf, p.region + static_cast<uint64_t>(i) * p.rec_pitch, p.x_row_bytes, bar);
            }
            int row = -1;
            if (p.do_expand && lane < K) {
                const int* mi = meta_of(i);
                const int e = mi[lane];
                if (e >= expert_begin && e < expert_begin + EL) row = mi[2 * K + lane];
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, i);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) break;
            if (!p.do_expand) {
                if (lane == 0 && i < p.num_out_rows) {
                    bulk_s2g(p.recv_x + static_cast<uint64_t>(i) * p.x_row_bytes, buf, p.x_row_bytes);
                    bulk_commit();
                }
            } else if (row >= 0 && row < p.num_out_rows) {
                bulk_s2g(p.recv_x + static_cast<uint64_t>(row) * p.x_row_bytes, buf, p.x_row_bytes);
                bulk_commit();
            }
        }
    }

    // ---- 4. zero the alignment gaps of the expanded layout
    if (p.do_expand && p.do_zero_padding) {
        const int vec_per_row = p.x_row_bytes / 16;
        for (int le = bid; le < EL; le += nb) {
            const int begin = p.psum_expert[le];                               // start + real count
            const int end = min(align_up(begin, p.expert_alignment), p.num_out_rows);
            for (int64_t v = static_cast<int64_t>(begin) * vec_per_row + tid; v < static_cast<int64_t>(end) * vec_per_row; v += nthreads)
                reinterpret_cast<int4*>(p.recv_x)[v] = make_int4(0, 0, 0, 0);
            if (p.recv_topk_weights != nullptr)
                for (int r = begin + tid; r < end; r += nthreads) p.recv_topk_weights[r] = 0.f;
            // the scales of the padding rows too: 0 x (whatever was in memory) would not be 0 for a NaN or an infinity
            if (p.recv_sf != nullptr && sf_packs > 0) {
                for (int i = tid; i < (end - begin) * sf_packs; i += nthreads) {
                    const int r = begin + i / sf_packs, k = i % sf_packs;
                    reinterpret_cast<uint32_t*>(p.recv_sf)[static_cast<int64_t>(r) * p.recv_sf_row_stride + static_cast<int64_t>(k) * p.recv_sf_pack_stride] = 0u;
                }
            }
        }
    }
    bulk_wait_all();
    if (bid == 0 && tid == 0) timeline[1] = globaltimer_ns();
}

}  // namespace

bool plan_dispatch(const DispatchParams& p, int num_sms, int smem_optin, DispatchLaunch* out) {
    const StageLayout sl = stage_layout(p.src_row_bytes, p.meta_bytes);
    const int avail = smem_optin - header_bytes(p.num_experts) - 128;   // 128: static shared memory of the kernel
    int warps = avail / sl.bytes;
    if (warps > 32) warps = 32;
    if (warps < 2) return false;
    // the ordering pass borrows the staging buffers: make sure one tile of routing words fits
    const int need = order_scratch_min_bytes(p.num_experts, p.num_topk, p.c.num_ranks);
    int scratch = warps * sl.bytes;
    if (scratch < need) scratch = align_up(need, 128);
    // At eight ranks the send phase is bound by NVLink, and every send warp beyond what saturates the wire only
    // lengthens the queue in front of it: a warp holds one token (about 40 KB over its destinations), the queue drains
    // at the wire's rate, and what is queued when the tokens run out is the tail of the kernel (measured at EP8 with
    // 24 SMs: 360 tokens in flight = 17 us with the cast fused, 720 tokens = 29 us with pre-quantised input). About
    // 200 tokens in flight per rank keep the wire busy; the cast needs a few more warps to hide its latency. (With
    // four ranks a quarter of the rows stays local and the cast needs the warps: no cap there.)
    if (p.c.num_ranks >= 8) {
        const int target = p.quant_mode != kQuantNone ? 256 : 192;
        int cap = ceil_div(target, num_sms);
        if (cap < 4) cap = 4;
        if (warps > cap) warps = cap;
    }
    if (scratch > avail) return false;
    out->num_sms = num_sms;
    out->num_warps = warps;
    out->scratch_bytes = scratch;
    out->smem_bytes = header_bytes(p.num_experts) + scratch;
    return true;
}

cudaError_t launch_dispatch(const Multi<DispatchParams>& m, const DispatchLaunch& l, cudaStream_t stream) {
    cudaError_t err = prepare_kernel(dispatch_kernel, l.smem_bytes);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m.num_vranks * m.blocks_per_rank);
    cfg.blockDim = dim3(l.num_warps * 32);
    cfg.dynamicSmemBytes = l.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    Multi<DispatchParams> copy = m;
    for (int v = 0; v < copy.num_vranks; ++v) copy.r[v].smem_scratch_bytes = l.scratch_bytes;
    return cudaLaunchKernelEx(&cfg, dispatch_kernel, copy);
}

cudaError_t launch_dispatch_epilogue(const DispatchEpilogueParams* params, int num_vranks, int num_sms, int smem_optin,
                                     cudaStream_t stream, bool programmatic) {
    Multi<DispatchEpilogueParams> m;
    m.num_vranks = num_vranks;
    m.blocks_per_rank = num_sms;
    for (int v = 0; v < num_vranks; ++v) m.r[v] = params[v];
    const bool move_rows = params[0].copy_x || params[0].do_expand;
    const int stage = align_up(params[0].x_row_bytes, 128) + 16;
    int warps = move_rows ? smem_optin / stage : 32;
    if (warps > (move_rows ? 16 : 32)) warps = move_rows ? 16 : 32;
    if (warps < 1) return cudaErrorInvalidValue;
    const int smem_bytes = move_rows ? warps * stage : 0;
    cudaError_t err = prepare_kernel(dispatch_epilogue_kernel, smem_bytes);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_vranks * num_sms);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dispatch_epilogue_kernel, m);
}

}  // namespace ep
