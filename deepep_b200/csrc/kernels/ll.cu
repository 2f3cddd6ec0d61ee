// Low-latency expert-parallel dispatch / combine for decode batches (sm_100a, NVLink only).
//
// Dispatch, SEND phase: one thread block per token (round-robin). The block casts the bf16 row
// to e4m3 with 1x128 scales (optionally power-of-two scales, optionally packed as UE8M0) into a
// shared-memory message, then one warp per selected expert bulk-stores the message into slot
// [local expert][source rank][position] of the owner's receive area. Positions are the token's
// rank among this source's earlier tokens for that expert, so they do not depend on timing.
// Every message carries its own arrival flag: its 8-byte header (call number, token, top-k lane)
// is written last. The sending warps wait until wait_group has confirmed their payload and meet
// one more warp at a named barrier; that warp issues ONE release fence at system scope for the
// token and writes the K headers (a fence per message was measured at 7 us when the warps of an
// SM issue them side by side, a full async-proxy fence at 5 us; with no fence at all a header
// can overtake its payload on NVLink, which showed up as rows packed before they had landed on
// 4 GPUs). The rest of the block casts the next token meanwhile. The per-expert counts need no
// data at all (they come from the routing), so they travel first, as call-tagged words, while
// the payloads are cast.
// Dispatch, RECV phase: one block per (local expert, source rank) waits for the counts of the
// sources before it (prefix) and then, message by message, for the header of each slot; rows are
// packed expert-major as they land: grouped by source rank in ascending order, scales
// column-major, plus src_info / layout_range / recv_count for the combine.
//
// Combine, SEND phase: every packed row goes back to row [top-k lane][token] of its source
// rank's combine area (the lane travelled with the token, which keeps the area at
// lanes x tokens rows, small enough to stay in L2). A block sends its rows in rounds of one row
// per warp; behind each round one thread issues the system-scope release fence for the whole
// block and every warp then writes the call-tagged flag word of its (lane, token). Combine, RECV
// phase: per token, wait for the flags of its own rows only, accumulate sum_k w_k * row_k in
// fp32 in ascending lane order, round to bf16 once. Nothing is counted and nothing has to be
// cleared between calls.
//
// No host synchronisation, no launch parameter that changes from call to call: the call
// counters that select the buffer half and tag the flags live in device memory, so a captured
// CUDA graph replays correctly. SEND and RECV can be launched separately (receive hooks).
//
// Parity: csrc/kernels/legacy/internode_ll.cu:128-462 (dispatch), :714-1138 (combine),
// :21-126 and :1240-1285 (clean / mask) of the reference.
#include <cstdlib>

#include "api.hpp"
#include "../common/device_utils.cuh"

namespace ep {

namespace {

__device__ __forceinline__ int* ll_ints(const CommCtx& c) {
    return reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsLLOffsetBytes);
}
__device__ __forceinline__ int* ll_mask(const CommCtx& c) { return ll_ints(c) + 2 * kMaxExperts; }
__device__ __forceinline__ int* ll_done(const CommCtx& c) { return ll_ints(c) + 2 * kMaxExperts + kMaxRanks; }

__device__ __forceinline__ int ld_volatile_int(const int* p) {
    return *reinterpret_cast<const volatile int*>(p);
}

// Last block of a phase advances that phase's call counter (all blocks have read it by then).
__device__ __forceinline__ void ll_phase_done(const CommCtx& c, int phase_idx, int nb) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const int old = atomicAdd(ll_done(c) + phase_idx, 1);
        if (old == nb - 1) {
            ll_done(c)[phase_idx] = 0;
            __threadfence();
            atomicAdd(reinterpret_cast<unsigned long long*>(c.local_ws + kWsLLCalls + phase_idx), 1ull);
        }
    }
}

// A wait that either reports (normal mode) or masks the silent peer (shrink mode).

// -------------------------------------------------------------------- LogFMT-10 (combine wire format)
// Per group of 128 channels the sender records amax and amin of |x| (bf16). If amax < 1 and amin < amax, every value
// becomes a sign bit and a 9-bit code on a logarithmic grid between amin and amax: code 0 is zero, code c >= 1 is
// 2^(log_amin + (c - 1) * step) with step = (log_amax - log_amin) / 510, log_amin clipped to log_amax - 32. Sixteen
// values pack into 160 bits (codes first, the sixteen sign bits last). Groups that do not qualify stay bf16. The
// receiver redoes the same arithmetic on the same two bf16 numbers, so both sides agree on which groups were cast.
// Same format and thresholds as csrc/kernels/legacy/internode_ll.cu:556-712 of the reference.
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct LogFmtGroup {
    float log_amin, step;
    bool cast;
};

__device__ __forceinline__ LogFmtGroup logfmt_group(float amax, float amin) {
    LogFmtGroup q;
    const float la = lg2_approx(amax);
    q.log_amin = fmaxf(lg2_approx(amin), la - 32.f);
    q.cast = la < 0.f && q.log_amin < la;
    q.step = (la - q.log_amin) * (1.f / 510.f);
    return q;
}

// Sixteen bf16 values (eight packed words) -> five words.
__device__ __forceinline__ void logfmt_pack16(const uint32_t* v, float log_amin, float step_inv, float rounding, uint32_t* out) {
    uint64_t acc = 0;
    int nbits = 0, w = 0;
    uint32_t signs = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        signs |= ((v[i] >> 15) & 1u) << (2 * i) | ((v[i] >> 31) & 1u) << (2 * i + 1);
        const uint32_t a = v[i] & 0x7fff7fffu;
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float mag = h == 0 ? f.x : f.y;
            const uint32_t code = __float2uint_rd(fmaxf((lg2_approx(mag) - log_amin) * step_inv + rounding, 0.f));
            acc |= static_cast<uint64_t>(code) << nbits;
            nbits += 9;
            if (nbits >= 32) {
                out[w++] = static_cast<uint32_t>(acc);
                acc >>= 32;
                nbits -= 32;
            }
        }
    }
    out[4] = static_cast<uint32_t>(acc) | (signs << 16);   // 16 bits of codes are left, the signs fill the word
}

// acc[16] += weight * decoded value, from five words.
__device__ __forceinline__ void logfmt_unpack16_fma(const uint32_t* in, float log_amin, float step, float weight, float* acc) {
    const uint32_t signs = in[4] >> 16;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int bit = 9 * i, w = bit >> 5, sh = bit & 31;
        const uint32_t code = (sh + 9 <= 32 ? in[w] >> sh : __funnelshift_r(in[w], in[w + 1], sh)) & 0x1ffu;
        float val = code == 0 ? 0.f : ex2_approx(static_cast<float>(code - 1) * step + log_amin);
        if ((signs >> i) & 1u) val = -val;
        acc[i] = fmaf(weight, val, acc[i]);
    }
}

// Warp-collective: encodes the bf16 row at `payload` in place and fills `meta`; returns the packed payload bytes.
// Eight groups per pass, 32 channels per lane (four lanes share a group). Every lane holds its 32 channels in
// registers before any lane writes, and the output of a pass never reaches the input of the next one.
__device__ __forceinline__ int logfmt_encode_row(uint8_t* meta, uint8_t* payload, int hidden, int lane) {
    const int G = hidden / 128;
    int packed = 0;
    for (int b = 0; b * 8 < G; ++b) {
        const int g = b * 8 + (lane >> 2);
        const bool valid = g < G;
        uint32_t v[16];
        if (valid) {
            const int4* src = reinterpret_cast<const int4*>(payload + (static_cast<size_t>(b) * 1024 + lane * 32) * 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<int4*>(v + 4 * i) = src[i];
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0;
        }
        __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.f, 0.f);
        uint32_t inf2 = 0x7f807f80u;
        __nv_bfloat162 amin2 = *reinterpret_cast<__nv_bfloat162*>(&inf2);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t a = v[i] & 0x7fff7fffu;
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&a);
            amax2 = __hmax2(amax2, h);
            amin2 = __hmin2(amin2, h);
        }
        float amax = fmaxf(__low2float(amax2), __high2float(amax2));
        float amin = fminf(__low2float(amin2), __high2float(amin2));
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            amin = fminf(amin, __shfl_xor_sync(0xffffffffu, amin, o));
        }
        const LogFmtGroup q = logfmt_group(amax, amin);
        const bool cast = valid && q.cast;
        if (valid && (lane & 3) == 0) {
            const __nv_bfloat162 mm = __floats2bfloat162_rn(amax, amin);
            reinterpret_cast<uint32_t*>(meta)[g] = *reinterpret_cast<const uint32_t*>(&mm);
        }
        const unsigned cast_mask = __ballot_sync(0xffffffffu, cast);
        const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
        const int off = packed + lane * 64 - 24 * __popc(cast_mask & ((1u << lane) - 1u));
        __syncwarp();
        if (valid) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(payload + off);
            if (cast) {
                const float step_inv = 1.f / q.step;
                const float rounding = 2.f - lg2_approx((1.f + ex2_approx(q.step)) * 0.5f) * step_inv;
                uint32_t out[10];
                logfmt_pack16(v, q.log_amin, step_inv, rounding, out);
                logfmt_pack16(v + 8, q.log_amin, step_inv, rounding, out + 5);
#pragma unroll
                for (int i = 0; i < 5; ++i) *reinterpret_cast<uint2*>(dst + 2 * i) = make_uint2(out[2 * i], out[2 * i + 1]);
            } else if (off != (b * 1024 + lane * 32) * 2) {
#pragma unroll
                for (int i = 0; i < 8; ++i) *reinterpret_cast<uint2*>(dst + 2 * i) = make_uint2(v[2 * i], v[2 * i + 1]);
            }
        }
        packed += __popc(valid_mask) * 64 - 24 * __popc(cast_mask);
        __syncwarp();
    }
    return packed;
}

template <typename Pred>
__device__ __forceinline__ bool ll_wait(const WaitCtx& w, const CommCtx& c, int shrink, int code, int peer, uint32_t tag, Pred pred) {
    if (!shrink) return bounded_wait(w, code, peer, tag, pred);
    uint32_t spins = 0;
    while (!pred()) {
        if ((++spins & 63u) == 0) {
            if (ld_volatile_int(ll_mask(c) + peer) != 0) return false;
            if (globaltimer_ns() > w.deadline_ns) {
                atomicExch(ll_mask(c) + peer, 1);
                return false;
            }
        }
    }
    return true;
}

// ==================================================================== dispatch
__global__ void __launch_bounds__(1024, 1) ll_dispatch_kernel(const __grid_constant__ Multi<LLDispatchParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const LLDispatchParams& p = m.r[vr];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int num_warps = blockDim.x >> 5;
    const int T = p.num_tokens, H = p.hidden, K = p.num_topk, E = p.num_experts, EL = p.num_local_experts;
    const int R = c.num_ranks, Tm = p.num_max_tokens;
    const int msg_bytes = ll_dispatch_msg_bytes(H, p.use_fp8);
    const int payload_bytes = p.use_fp8 ? H : H * 2;
    const int* mask = ll_mask(c);
    uint64_t* stamps = c.local_ws + kWsStamps;          // phase timestamps of block 0 (ns), read by the profiling helpers
    const bool stamper = bid == 0 && tid == 0;
    // launched as a programmatic dependent: resident early, but nothing is touched before the kernel ahead has finished
    dependency_wait();
    launch_dependents();
    if (stamper) stamps[0] = globaltimer_ns();

    if (p.phases & kLLSend) {
        const uint32_t epoch = static_cast<uint32_t>(*reinterpret_cast<volatile uint64_t*>(c.local_ws + kWsLLCalls + 0)) + 1;
        const int half = epoch & 1;
        int* s_topk = reinterpret_cast<int*>(smem);                         // [T * K]
        uint8_t* s_msg = smem + align_up(T * K * 4, 128);                   // [2][msg_bytes aligned]
        const int msg_stride = align_up(msg_bytes, 128);
        // the first row's load is issued before the routing is read: two independent trips to memory overlap
        int4 first_raw = make_int4(0, 0, 0, 0);
        if (bid < T && tid * 8 < H) first_raw = ld_nc_int4(p.x + (static_cast<int64_t>(bid) * H + tid * 8) * 2);
        for (int i = tid; i < T * K; i += blockDim.x) {
            s_topk[i] = load_topk_idx(p.topk_idx, p.idx32 != 0, i, E);
        }
        __syncthreads();

        // ---- the per-expert counts first: they depend on the routing only
        // (by the warps that do not send, while the others cast and send)
        const int num_publishers = num_warps > K ? num_warps - K : num_warps;
        auto publish_counts = [&](int pw) {
            for (int e = bid + pw * nb; e < E; e += nb * num_publishers) {
                const int dst = e / EL;
                if (ld_volatile_int(mask + dst) != 0) continue;
                int total = 0;
                for (int i = lane; i < T * K; i += 32) total += s_topk[i] == e;
                total = warp_reduce_sum(total);
                if (lane == 0) {
                    uint64_t* word = reinterpret_cast<uint64_t*>(c.heap[dst] + p.off_recv_count[half]) + (e - dst * EL) * R + c.rank;
                    st_release_sys_u64(word, pack_epoch(epoch, static_cast<uint32_t>(total)));
                }
            }
        };
        if (num_warps > K && warp >= K) publish_counts(warp - K);

        int iter = 0;
        // Headers (= arrival flags) of the K messages of a token: the sending warps park them here once wait_group has
        // confirmed their payload; warp K then issues ONE release fence at system scope for the whole token and writes the
        // K headers. (A fence per message costs microseconds apiece when the warps of an SM issue them side by side; a
        // plain store behind wait_group is not enough: over NVLink the small header can overtake its payload.)
        __shared__ uint64_t* s_hdr[kMaxLLTopk];
        __shared__ uint64_t s_hval[kMaxLLTopk];
        for (int t = bid; t < T; t += nb, ++iter) {
            uint8_t* msg = s_msg + (iter & 1) * msg_stride;
            uint8_t* payload = msg + 16;
            // ---- cast / copy the row into the message
            const int ch = tid * 8;
            const bool active = ch < H;
            int4 raw = first_raw;
            if (active && iter != 0) raw = ld_nc_int4(p.x + (static_cast<int64_t>(t) * H + ch) * 2);
            if (!p.use_fp8) {
                if (active) *reinterpret_cast<int4*>(payload + ch * 2) = raw;
            } else {
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                float f[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 v = __bfloat1622float2(h2[i]);
                    f[2 * i] = v.x;
                    f[2 * i + 1] = v.y;
                }
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
                // every thread takes part in the shuffles (inactive lanes carry zeros); hidden % 128 == 0,
                // so a 16-lane scale group is either all active or all inactive
                amax = warp_reduce_max_width(amax, 16);
                float scale, inv;
                fp8_scale_from_amax(amax, p.round_scale != 0, scale, inv);
                uint2 packed;
                packed.x = pack4_e4m3(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
                packed.y = pack4_e4m3(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
                if (active) {
                    *reinterpret_cast<uint2*>(payload + ch) = packed;
                    if ((lane & 15) == 0) {
                        if (p.use_ue8m0) payload[H + (ch >> 7)] = static_cast<uint8_t>(__float_as_uint(scale) >> 23);
                        else reinterpret_cast<float*>(payload + H)[ch >> 7] = scale;
                    }
                }
            }
            fence_proxy_async_smem();
            __syncthreads();   // message complete; also: the stores of two tokens ago have finished reading this buffer
            // ---- one warp per selected expert
            if (warp < K) {
                const int e = s_topk[t * K + warp];
                const int dst = e >= 0 ? e / EL : -1;
                const bool send = e >= 0 && ld_volatile_int(mask + dst) == 0;
                int slot = 0;
                if (send) {
                    int before = 0;
                    for (int i = lane; i < t * K; i += 32) before += s_topk[i] == e;
                    slot = warp_reduce_sum(before);
                }
                if (lane == 0) {
                    uint64_t* hdr = nullptr;
                    if (send) {
                        uint8_t* dst_msg = c.heap[dst] + p.off_recv_x[half] +
                                           ((static_cast<uint64_t>(e - dst * EL) * R + c.rank) * Tm + slot) * msg_bytes;
                        bulk_s2g(dst_msg + 16, payload, msg_bytes - 16);
                        bulk_commit();
                        bulk_wait_all();
                        hdr = reinterpret_cast<uint64_t*>(dst_msg);
                    }
                    s_hdr[warp] = hdr;
                    s_hval[warp] = pack_epoch(epoch, static_cast<uint32_t>(t | (warp << 16)));
                }
                __syncwarp();
            }
            if (warp <= K) {
                // warps 0..K-1 have their stores confirmed, warp K raises the flags behind one fence
                asm volatile("bar.sync 1, %0;" ::"r"((K + 1) * 32) : "memory");
                if (warp == K) {
                    if (lane == 0) fence_acq_rel_sys();
                    __syncwarp();
                    if (lane < K && s_hdr[lane] != nullptr) st_relaxed_sys_u64(s_hdr[lane], s_hval[lane]);
                }
            }
        }
        if (num_warps <= K) publish_counts(warp);
        if (stamper) stamps[1] = globaltimer_ns();
        if (stamper) stamps[2] = globaltimer_ns();
        ll_phase_done(c, 0, nb);
        if (stamper) stamps[3] = globaltimer_ns();
    }

    if (p.phases & kLLRecv) {
        const uint32_t epoch = static_cast<uint32_t>(*reinterpret_cast<volatile uint64_t*>(c.local_ws + kWsLLCalls + 1)) + 1;
        const int half = epoch & 1;
        // Work item = (local expert, source rank). A block takes its items in rounds of up to kRound: first the count
        // words of all sources of those experts (the rows of a source start behind the rows of the sources before it),
        // all in parallel, then -- without another block-wide barrier -- the rows of its own sources, a row cut into
        // kParts pieces of one warp each so that the few rows of an item keep every warp busy.
        constexpr int kRound = 8, kParts = 8;
        __shared__ int s_cnt[kRound][kMaxRanks], s_begin[kRound][kMaxRanks];
        const int rows_per_expert = R * Tm;
        const int sf_per_row = p.use_fp8 ? (p.use_ue8m0 ? H / 512 : H / 128) : 0;
        const int vec_per_part = ceil_div(payload_bytes / 16, kParts);
        for (int item0 = bid; item0 < EL * R; item0 += nb * kRound) {
            int n_items = 0;
            while (n_items < kRound && item0 + n_items * nb < EL * R) ++n_items;
            __syncthreads();
            for (int q = tid; q < n_items * R; q += blockDim.x) {
                const int it = q / R, s = q % R;
                const int le = (item0 + it * nb) / R;
                int cnt = 0;
                if (ld_volatile_int(mask + s) == 0) {
                    const uint64_t* word = reinterpret_cast<const uint64_t*>(c.heap[c.rank] + p.off_recv_count[half]) + le * R + s;
                    uint64_t v = 0;
                    const bool ok = ll_wait(w, c, p.shrink, kStatusLLRecv, s, le, [&]() {
                        v = ld_acquire_sys_u64(word);
                        return epoch_matches(v, epoch);
                    });
                    if (ok) cnt = static_cast<int>(static_cast<uint32_t>(v));
                }
                s_cnt[it][s] = cnt;
            }
            __syncthreads();
            if (tid < n_items) {
                const int item = item0 + tid * nb, le = item / R, src_rank = item % R;
                int acc = 0;
                for (int s = 0; s < R; ++s) {
                    s_begin[tid][s] = acc;
                    if (src_rank == 0)
                        p.packed_recv_layout_range[le * R + s] = (static_cast<int64_t>(acc) << 32) | static_cast<uint32_t>(s_cnt[tid][s]);
                    acc += s_cnt[tid][s];
                }
                if (src_rank == 0) {
                    p.packed_recv_count[le] = acc;
                    if (p.cumulative_stats != nullptr) atomicAdd(p.cumulative_stats + le, acc);
                }
            }
            __syncthreads();
            for (int it = 0; it < n_items; ++it) {
                const int item = item0 + it * nb, le = item / R, src_rank = item % R;
                const int begin = s_begin[it][src_rank], count = s_cnt[it][src_rank];
                for (int u = warp; u < count * kParts; u += num_warps) {
                    const int slot = u / kParts, part = u % kParts;
                    const int j = begin + slot;
                    const uint8_t* src = c.heap[c.rank] + p.off_recv_x[half] + ((static_cast<uint64_t>(le) * R + src_rank) * Tm + slot) * msg_bytes;
                    const int64_t out_row = static_cast<int64_t>(le) * rows_per_expert + j;
                    // the header is the message's arrival flag: written last by the sender, tagged with the call number
                    uint64_t hdr = 0;
                    const uint64_t t0 = (p.wait_stats != nullptr && lane == 0) ? globaltimer_ns() : 0;
                    const bool landed = ll_wait(w, c, p.shrink, kStatusLLRecv, src_rank, le, [&]() {
                        hdr = ld_acquire_sys_u64(reinterpret_cast<const uint64_t*>(src));
                        return epoch_matches(hdr, epoch);
                    });
                    if (!__all_sync(0xffffffffu, landed)) break;      // reported, or the source is masked now: its rows stay unwritten
                    if (lane == 0 && part == 0) {
                        p.packed_recv_src_info[out_row] = static_cast<int>(static_cast<uint32_t>(hdr));
                        if (p.wait_stats != nullptr) atomicAdd(reinterpret_cast<unsigned long long*>(p.wait_stats + src_rank), globaltimer_ns() - t0);
                    }
                    uint8_t* dst = p.packed_recv_x + out_row * payload_bytes;
                    const int v_end = min(payload_bytes / 16, (part + 1) * vec_per_part);
                    for (int v = part * vec_per_part + lane; v < v_end; v += 32 * 4) {   // four loads in flight per lane
                        int4 tmp[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (v + 32 * q < v_end) tmp[q] = ld_nc_int4(src + 16 + (v + 32 * q) * 16);
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (v + 32 * q < v_end) st_na_int4(dst + (v + 32 * q) * 16, tmp[q]);
                    }
                    if (sf_per_row > 0 && part == kParts - 1) {
                        const uint32_t* sf = reinterpret_cast<const uint32_t*>(src + 16 + H);
                        uint32_t* out_sf = reinterpret_cast<uint32_t*>(p.packed_recv_sf);
                        for (int i = lane; i < sf_per_row; i += 32)
                            out_sf[(static_cast<int64_t>(le) * sf_per_row + i) * rows_per_expert + j] = sf[i];
                    }
                }
            }
        }
        if (stamper) stamps[4] = globaltimer_ns();
        ll_phase_done(c, 1, nb);
        if (stamper) stamps[5] = globaltimer_ns();
    }
}

// ==================================================================== combine
__global__ void __launch_bounds__(512, 1) ll_combine_kernel(const __grid_constant__ Multi<LLCombineParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank;
    const int nb = m.blocks_per_rank;
    const LLCombineParams& p = m.r[vr];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();
    const int num_warps = blockDim.x >> 5;
    const int T = p.num_tokens, H = p.hidden, K = p.num_topk, E = p.num_experts, EL = p.num_local_experts;
    const int R = c.num_ranks, Tm = p.num_max_tokens;
    const int row_bytes = H * 2;
    const int meta_bytes = p.use_logfmt ? ll_logfmt_meta_bytes(H) : 0;
    const int slot_bytes = row_bytes + meta_bytes;
    const int* mask = ll_mask(c);
    dependency_wait();
    launch_dependents();
    // phase timestamps of block 0 (ns): start, rows issued, flags raised, send phase handed over, tokens reduced, end
    uint64_t* stamps = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(c.local_ws) + kWsTimelineOffsetBytes) + 8;
    const bool stamper = bid == 0 && tid == 0;
    if (stamper) stamps[0] = globaltimer_ns();

    if (p.phases & kLLSend) {
        const uint32_t epoch = static_cast<uint32_t>(*reinterpret_cast<volatile uint64_t*>(c.local_ws + kWsLLCalls + 2)) + 1;
        const int half = epoch & 1;
        __shared__ int s_pref[kMaxLocalExperts + 1];
        // rows per local expert (begin + count of the last source rank), prefix-summed by warp 0
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < EL; base += 32) {
                const int le = base + lane;
                int rows = 0;
                if (le < EL) {
                    const int64_t last = p.layout_range[le * R + R - 1];
                    rows = static_cast<int>(last >> 32) + static_cast<int>(last & 0xffffffff);
                }
                int incl = rows;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                if (le < EL) s_pref[le] = carry + incl - rows;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) s_pref[EL] = carry;
        }
        __syncthreads();
        const int total_rows = s_pref[EL];
        const int stage = meta_bytes + align_up(row_bytes, 128) + 16;
        uint8_t* buf = smem + static_cast<size_t>(warp) * stage;   // [meta table (LogFMT only)][row]
        uint8_t* payload = buf + meta_bytes;
        uint64_t* bar = reinterpret_cast<uint64_t*>(payload + align_up(row_bytes, 128));
        if (lane == 0) {
            mbar_init(bar, 1);
            fence_mbar_init();
        }
        __syncwarp();
        uint32_t parity = 0;
        // Rows are taken in rounds (one row per warp and round). Per round: every warp stores its row and waits until
        // wait_group has confirmed it, the block meets, ONE thread issues a release fence at system scope, the block
        // meets again and every warp raises the flag of its row. (A fence per row costs microseconds apiece when the
        // warps of an SM issue them side by side; without any fence the flag can overtake its row on NVLink.)
        __shared__ int s_alive;
        if (tid == 0) s_alive = 1;
        __syncthreads();
        const int my_rows = max(total_rows - bid * num_warps, 0);
        const int rounds = ceil_div(my_rows, nb * num_warps);
        // sends row g if there is one for this warp; returns the address of its flag (lane 0), null if nothing was sent
        auto send_row = [&](int g) -> uint64_t* {
            if (g >= total_rows) return nullptr;
            int le = 0;
            {   // largest le with s_pref[le] <= g
                int lo = 0, hi = EL - 1;
                while (lo < hi) {
                    const int mid = (lo + hi + 1) >> 1;
                    if (s_pref[mid] <= g) lo = mid; else hi = mid - 1;
                }
                le = lo;
            }
            const int j = g - s_pref[le];
            int s = 0;
            while (s < R - 1 && j >= static_cast<int>(p.layout_range[le * R + s + 1] >> 32)) ++s;
            if (ld_volatile_int(mask + s) != 0) return nullptr;
            const int64_t row = static_cast<int64_t>(le) * R * Tm + j;
            const int info = p.src_info[row];
            const int token = info & 0xffff, k = info >> 16;
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, row_bytes);
                bulk_g2s(payload, p.x + row * row_bytes, row_bytes, bar);
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, g);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) {
                if (lane == 0) s_alive = 0;       // reported; the block stops after this round
                return nullptr;
            }
            int send_bytes = row_bytes;
            if (p.use_logfmt) {
                send_bytes = meta_bytes + logfmt_encode_row(buf, payload, H, lane);
                fence_proxy_async_smem();
                __syncwarp();
            }
            uint64_t* flag = nullptr;
            if (lane == 0) {
                bulk_s2g(c.heap[s] + p.off_combine_x[half] + (static_cast<uint64_t>(k) * Tm + token) * slot_bytes, buf, send_bytes);
                bulk_commit();
                bulk_wait_all();
                flag = reinterpret_cast<uint64_t*>(c.heap[s] + p.off_combine_flag[half]) + static_cast<uint64_t>(k) * Tm + token;
            }
            return flag;
        };
        for (int r = 0; r < rounds; ++r) {
            uint64_t* flag = send_row((r * nb + bid) * num_warps + warp);
            if (stamper) stamps[1] = globaltimer_ns();
            __syncthreads();
            if (tid == 0) fence_acq_rel_sys();
            __syncthreads();
            if (lane == 0 && flag != nullptr) st_relaxed_sys_u64(flag, pack_epoch(epoch, 1));
            if (s_alive == 0) break;
        }
        if (stamper) stamps[2] = globaltimer_ns();
        ll_phase_done(c, 2, nb);
        if (stamper) stamps[3] = globaltimer_ns();
    }

    if (p.phases & kLLRecv) {
        const uint32_t epoch = static_cast<uint32_t>(*reinterpret_cast<volatile uint64_t*>(c.local_ws + kWsLLCalls + 3)) + 1;
        const int half = epoch & 1;
        __shared__ float s_w[kMaxTopk];
        __shared__ int s_ok[kMaxTopk];
        const uint8_t* region = c.heap[c.rank] + p.off_combine_x[half];
        for (int t = bid; t < T; t += nb) {
            __syncthreads();
            if (tid < K) {
                const int e = load_topk_idx(p.topk_idx, p.idx32 != 0, static_cast<int64_t>(t) * K + tid, E);
                int ok = 0;
                if (e >= 0 && ld_volatile_int(mask + e / EL) == 0) {
                    const uint64_t* word = reinterpret_cast<const uint64_t*>(c.heap[c.rank] + p.off_combine_flag[half]) + static_cast<uint64_t>(tid) * Tm + t;
                    const uint64_t t0 = globaltimer_ns();
                    ok = ll_wait(w, c, p.shrink, kStatusLLCombine, e / EL, e, [&]() { return epoch_matches(ld_acquire_sys_u64(word), epoch); });
                    if (p.wait_stats != nullptr) atomicAdd(reinterpret_cast<unsigned long long*>(p.wait_stats + e / EL), globaltimer_ns() - t0);
                }
                s_ok[tid] = ok;
                s_w[tid] = p.topk_weights[static_cast<int64_t>(t) * K + tid];
            }
            __syncthreads();
            if (p.use_logfmt) {
                // ---- per (lane, group): cast or not, grid parameters, byte offset of the group in the packed row
                const int G = H / 128;
                float* s_lmin = reinterpret_cast<float*>(smem);
                float* s_step = s_lmin + K * G;
                int* s_off = reinterpret_cast<int*>(s_step + K * G);
                for (int k = warp; k < K; k += num_warps) {
                    if (!s_ok[k]) continue;
                    const uint8_t* row = region + (static_cast<uint64_t>(k) * Tm + t) * slot_bytes;
                    int carry = 0;
                    for (int g0 = 0; g0 < G; g0 += 32) {
                        const int g = g0 + lane;
                        int size = 0;
                        if (g < G) {
                            const uint32_t mw = ld_nc_u32(row + g * 4);
                            const __nv_bfloat162 mm = *reinterpret_cast<const __nv_bfloat162*>(&mw);
                            const LogFmtGroup q = logfmt_group(__low2float(mm), __high2float(mm));
                            size = q.cast ? 160 : 256;
                            s_lmin[k * G + g] = q.log_amin;
                            s_step[k * G + g] = q.cast ? q.step : -1.f;
                        }
                        int incl = size;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const int up = __shfl_up_sync(0xffffffffu, incl, o);
                            if (lane >= o) incl += up;
                        }
                        if (g < G) s_off[k * G + g] = carry + incl - size;
                        carry += __shfl_sync(0xffffffffu, incl, 31);
                    }
                }
                __syncthreads();
                for (int u = tid; u < H / 16; u += blockDim.x) {     // sixteen channels per thread and pass
                    const int g = u >> 3, j = u & 7;
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                    for (int k0 = 0; k0 < K; k0 += 4) {              // four rows in flight, added in ascending lane order
                        uint32_t raw[4][8];
                        float step[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int k = k0 + q;
                            step[q] = 0.f;
                            if (k < K && s_ok[k]) {
                                const uint8_t* src = region + (static_cast<uint64_t>(k) * Tm + t) * slot_bytes + meta_bytes + s_off[k * G + g];
                                step[q] = s_step[k * G + g];
                                if (step[q] >= 0.f) {
#pragma unroll
                                    for (int i = 0; i < 5; ++i) raw[q][i] = ld_nc_u32(src + j * 20 + i * 4);
                                } else {
                                    *reinterpret_cast<int4*>(raw[q]) = ld_nc_int4(src + j * 32);
                                    *reinterpret_cast<int4*>(raw[q] + 4) = ld_nc_int4(src + j * 32 + 16);
                                }
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int k = k0 + q;
                            if (k < K && s_ok[k]) {
                                const float wk = s_w[k];
                                if (step[q] >= 0.f) {
                                    logfmt_unpack16_fma(raw[q], s_lmin[k * G + g], step[q], wk, acc);
                                } else {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) {
                                        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[q][i]));
                                        acc[2 * i] = fmaf(wk, v.x, acc[2 * i]);
                                        acc[2 * i + 1] = fmaf(wk, v.y, acc[2 * i + 1]);
                                    }
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        int4 out;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[h * 8 + 2 * i], acc[h * 8 + 2 * i + 1]);
                        st_na_int4(p.combined_x + (static_cast<int64_t>(t) * H + u * 16 + h * 8) * 2, out);
                    }
                }
                continue;
            }
            for (int ch = tid * 8; ch < H; ch += blockDim.x * 8) {
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                for (int k0 = 0; k0 < K; k0 += 8) {      // up to eight rows in flight, added in ascending lane order
                    int4 raw[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (k0 + u < K && s_ok[k0 + u])
                            raw[u] = ld_nc_int4(region + ((static_cast<uint64_t>(k0 + u) * Tm + t) * H + ch) * 2);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (k0 + u < K && s_ok[k0 + u]) {
                            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                            const float wk = s_w[k0 + u];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 v = __bfloat1622float2(h2[i]);
                                acc[2 * i] = fmaf(wk, v.x, acc[2 * i]);
                                acc[2 * i + 1] = fmaf(wk, v.y, acc[2 * i + 1]);
                            }
                        }
                    }
                }
                int4 out;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                st_na_int4(p.combined_x + (static_cast<int64_t>(t) * H + ch) * 2, out);
            }
        }
        if (stamper) stamps[4] = globaltimer_ns();
        ll_phase_done(c, 3, nb);
        if (stamper) stamps[5] = globaltimer_ns();
    }
}

__global__ void ll_mask_kernel(uint64_t* local_ws, int rank, int value, int* out, int num_ranks) {
    int* mask = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(local_ws) + kWsLLOffsetBytes) + 2 * kMaxExperts;
    if (out != nullptr) {
        if (threadIdx.x < num_ranks) out[threadIdx.x] = mask[threadIdx.x];
    } else if (rank < 0) {
        if (threadIdx.x < kMaxRanks) mask[threadIdx.x] = 0;
    } else if (threadIdx.x == 0) {
        mask[rank] = value;
    }
}

// Cooperative (all blocks resident: blocks of one rank wait for blocks of other ranks, which in turn may wait for blocks
// of this rank that would otherwise not be scheduled yet) and programmatic dependent (the grid may become resident while
// the kernel ahead of it in the stream drains; it calls dependency_wait() before it touches anything).
template <typename Params>
cudaError_t coop_launch(void (*fn)(const Multi<Params>), const Multi<Params>& m, int grid, int block, int smem, cudaStream_t stream) {
    static const bool plain = [] { const char* v = std::getenv("EP_LL_PLAIN_LAUNCH"); return v != nullptr && v[0] == '1'; }();
    static const bool no_pdl = [] { const char* v = std::getenv("EP_DISABLE_PDL"); return v != nullptr && v[0] == '1'; }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (!plain) {
        attr[n].id = cudaLaunchAttributeCooperative;
        attr[n].val.cooperative = 1;
        ++n;
    }
    if (!no_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, fn, m);
}

}  // namespace

cudaError_t launch_ll_dispatch(const Multi<LLDispatchParams>& m, int num_sms, cudaStream_t stream) {
    const LLDispatchParams& p = m.r[0];
    const int msg_stride = align_up(ll_dispatch_msg_bytes(p.hidden, p.use_fp8), 128);
    const int smem_bytes = align_up(p.num_max_tokens * p.num_topk * 4, 128) + 2 * msg_stride;
    cudaError_t err = prepare_kernel(ll_dispatch_kernel, smem_bytes);
    if (err != cudaSuccess) return err;
    Multi<LLDispatchParams> copy = m;
    copy.blocks_per_rank = num_sms;
    return coop_launch(ll_dispatch_kernel, copy, m.num_vranks * num_sms, 1024, smem_bytes, stream);
}

cudaError_t launch_ll_combine(const Multi<LLCombineParams>& m, int num_sms, int smem_optin, cudaStream_t stream) {
    const LLCombineParams& p = m.r[0];
    const int stage = (p.use_logfmt ? ll_logfmt_meta_bytes(p.hidden) : 0) + align_up(p.hidden * 2, 128) + 16;
    int warps = smem_optin / stage;
    if (warps > 16) warps = 16;   // 512 threads: the receive loop wants more than 64 registers per thread
    if (warps < 1) return cudaErrorInvalidValue;
    const int smem_bytes = warps * stage;
    // the receive phase of a LogFMT call keeps three words per (lane, group) in the same shared memory
    if (p.use_logfmt && p.num_topk * (p.hidden / 128) * 12 > smem_bytes) return cudaErrorInvalidValue;
    cudaError_t err = prepare_kernel(ll_combine_kernel, smem_bytes);
    if (err != cudaSuccess) return err;
    Multi<LLCombineParams> copy = m;
    copy.blocks_per_rank = num_sms;
    return coop_launch(ll_combine_kernel, copy, m.num_vranks * num_sms, warps * 32, smem_bytes, stream);
}

cudaError_t ll_update_mask(uint64_t* local_ws, int rank, int value, cudaStream_t stream) {
    ll_mask_kernel<<<1, 32, 0, stream>>>(local_ws, rank, value, nullptr, 0);
    return cudaGetLastError();
}

cudaError_t ll_query_mask(uint64_t* local_ws, int* out, int num_ranks, cudaStream_t stream) {
    ll_mask_kernel<<<1, 32, 0, stream>>>(local_ws, 0, 0, out, num_ranks);
    return cudaGetLastError();
}

}  // namespace ep
