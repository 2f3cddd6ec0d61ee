// Host/device shared definitions: limits, the per-rank communication context,
// status codes and the layout of the symmetric heap.
//
// The symmetric heap of a rank is one allocation that every peer of the NVLink
// domain maps into its own address space:
//
//   [0, kCtlBytes)            control words written by peers (epoch-tagged, never cleared)
//   [kCtlBytes, ...)          data regions, carved per operation by the functions below
//
// Parity: deep_ep/include/deep_ep/common/layout.cuh (WorkspaceLayout, TokenLayout,
// BufferLayout) and csrc/elastic/buffer.hpp:586-686 (buffer size calculators) in the
// reference. There is a single tier here (NVLink/NVSwitch), so the scale-out
// halves of those layouts have no counterpart.
#pragma once

#include <cstdint>
#include <cstddef>

#if defined(__CUDACC__)
#define EP_HD __host__ __device__ __forceinline__
#else
#define EP_HD inline
#endif

namespace ep {

// ---------------------------------------------------------------- limits
constexpr int kMaxRanks = 8;              // one NVSwitch domain of a B200 box
constexpr int kMaxExperts = 2048;
constexpr int kMaxLocalExperts = 256;
constexpr int kMaxTopk = 32;
constexpr int kMaxBlocks = 160;           // >= SM count of a B200 (148)
constexpr int kMaxVRanks = 8;             // ranks that one launch may emulate on a single GPU
constexpr int kMaxAgrsInflight = 32;
constexpr size_t kHeapAlignment = 2ull << 20;

template <typename T>
EP_HD constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }
template <typename T>
EP_HD constexpr T align_up(T a, T b) { return ceil_div(a, b) * b; }

// ---------------------------------------------------------------- status codes (first failure wins)
enum StatusCode : int {
    kStatusOk = 0,
    kStatusGridBarrier = 1,     // a block of this rank did not reach the grid barrier
    kStatusBarrierPeer = 2,     // a peer did not arrive at the cross-rank barrier
    kStatusDispatchCounts = 3,  // a peer's token counts did not arrive
    kStatusDispatchDone = 4,    // a peer did not finish its dispatch sends
    kStatusCombineDone = 5,     // a peer did not finish its combine sends
    kStatusTmaLoad = 6,         // a local bulk load did not complete
    kStatusLLRecv = 7,          // low-latency receive flag did not arrive
    kStatusLLCombine = 8,       // low-latency combine flag did not arrive
    kStatusEntry = 9,           // a peer did not enter the cached dispatch
    kStatusPP = 10,             // pipeline slot / arrival signal did not arrive
    kStatusAgrs = 11,           // all-gather arrival flag did not arrive
    kStatusGemmPipe = 12,       // a GEMM pipeline barrier did not complete
    kStatusTileFlag = 13,       // a fused GEMM+collective tile flag did not arrive
};

// ---------------------------------------------------------------- private (per-rank, not peer-mapped) workspace, in uint64 words
constexpr int kWsGridBarrier = 0;    // monotonically growing arrival counter
constexpr int kWsPoison = 1;         // non-zero after any wait of this rank gave up
constexpr int kWsStamps = 2;         // [8] phase timestamps of the last dispatch (ns): start, counted, ordered, totals in, bases
                                     // published, last row issued (all of block 0), own stores complete, all blocks done
constexpr int kWsWork = 10;          // next token index handed out by the dynamic send loops
constexpr int kWsLLCalls = 11;       // [4] low-latency call counters: dispatch send, dispatch recv, combine send, combine recv
constexpr int kWsScratch = 16;       // start of per-block scratch counters
// scratch: int32 [kMaxBlocks][kMaxRanks + kMaxExperts]
constexpr size_t kWsScratchInts = static_cast<size_t>(kMaxBlocks) * (kMaxRanks + kMaxExperts);
// low-latency area (int32): [2 * kMaxExperts] unused, [kMaxRanks] rank mask, [4] blocks-done counters of the four phases
constexpr size_t kWsLLOffsetBytes = kWsScratch * 8 + kWsScratchInts * 4;
constexpr size_t kWsLLInts = 2 * kMaxExperts + kMaxRanks + 4;
// tensor-parallel fused operators (int32): [64 chunks][kMaxRanks] rows-landed counters of the all-gather push
constexpr size_t kWsTpOffsetBytes = kWsLLOffsetBytes + kWsLLInts * 4;
constexpr size_t kWsTpInts = 64 * kMaxRanks;
// dispatch work sharing (int32): [kMaxBlocks] next token of every block's chunk, [kMaxBlocks] "bases published" epochs,
// [kMaxBlocks][kMaxRanks + kMaxExperts] the published first rows of every block's chunk
constexpr size_t kWsStealOffsetBytes = kWsTpOffsetBytes + kWsTpInts * 4;
constexpr size_t kWsStealInts = 2 * static_cast<size_t>(kMaxBlocks) + static_cast<size_t>(kMaxBlocks) * (kMaxRanks + kMaxExperts);
// kernel timeline (uint64 ns, %globaltimer): [8 kernels][start of block 0, end of the last block to leave]
constexpr size_t kWsTimelineOffsetBytes = align_up<size_t>(kWsStealOffsetBytes + kWsStealInts * 4, 8);
constexpr int kTlDispatch = 0, kTlDispatchEpilogue = 1, kTlCombine = 2, kTlCombineReduce = 3;
constexpr size_t kWsBytes = kWsTimelineOffsetBytes + 16 * 8 + 4096;

// ---------------------------------------------------------------- control area of the symmetric heap, in uint64 words
constexpr size_t kCtlBarrier = 0;                                        // [kMaxRanks]
constexpr size_t kCtlDispatchEntry = kCtlBarrier + kMaxRanks;            // [kMaxRanks]
constexpr size_t kCtlDispatchDone = kCtlDispatchEntry + kMaxRanks;       // [kMaxRanks]
constexpr size_t kCtlCombineDone = kCtlDispatchDone + kMaxRanks;         // [kMaxRanks]
constexpr size_t kCtlPPSignals = kCtlCombineDone + kMaxRanks;            // [2 dirs][2 kinds][64 slots]
constexpr size_t kCtlAgrsSignals = kCtlPPSignals + 256;                  // [kMaxAgrsInflight + 1][kMaxRanks]
constexpr size_t kCtlTileFlags = kCtlAgrsSignals + (kMaxAgrsInflight + 1) * kMaxRanks;  // [kMaxRanks][64]
constexpr size_t kCtlDispatchCnt = kCtlTileFlags + kMaxRanks * 64;       // [kMaxRanks][kMaxRanks + kMaxExperts]
constexpr size_t kCtlWords = kCtlDispatchCnt + static_cast<size_t>(kMaxRanks) * (kMaxRanks + kMaxExperts);
constexpr size_t kCtlBytes = align_up<size_t>(kCtlWords * 8, kHeapAlignment);

// ---------------------------------------------------------------- per-rank communication context passed to every kernel
struct CommCtx {
    int rank;
    int num_ranks;
    uint8_t* heap[kMaxRanks];   // heap[r] = base of rank r's symmetric heap in this rank's address space
    uint64_t* local_ws;         // private workspace (kWs* indices)
    uint64_t* host_status;      // mapped pinned host words: [0] failure record
    uint64_t timeout_ns;
};

// One launch can carry several virtual ranks (blocks [v*bpr, (v+1)*bpr) act as rank v);
// production launches carry exactly one.
template <typename P>
struct Multi {
    int num_vranks;
    int blocks_per_rank;
    P r[kMaxVRanks];
};

// ---------------------------------------------------------------- high-throughput EP layout
// One record travels per (token, destination rank), as ONE bulk store:
//   [payload row][scale factors][topk idx int32 x K][topk weights f32 x K][expanded rows int32 x K][src token int32][pad]
// The part after the payload is the "meta" of the record. Records sit `pitch` bytes apart in the receive
// region (a multiple of 128, so every record starts on a full NVLink packet / cache line); payload and
// scale factors are handed to the caller as strided views when it asks for zero copy.
EP_HD int ht_meta_bytes(int sf_bytes, int num_topk) {
    return static_cast<int>(align_up<int>(sf_bytes + 12 * num_topk + 4, 16));
}
EP_HD int ht_meta_bytes_max(int hidden, int num_topk) {
    return ht_meta_bytes(ceil_div(hidden, 128) * 4, num_topk);
}
EP_HD int ht_record_bytes(int x_row_bytes, int sf_bytes, int num_topk) { return x_row_bytes + ht_meta_bytes(sf_bytes, num_topk); }
EP_HD int ht_record_pitch(int x_row_bytes, int sf_bytes, int num_topk) {
    return align_up<int>(ht_record_bytes(x_row_bytes, sf_bytes, num_topk), 128);
}

// rows per arrival counter of the combine (arrival-driven reduce)
constexpr int kCombineFlagRows = 32;

struct HtLayout {
    // all offsets are bytes from the heap base
    uint64_t dispatch_rec[2];  // [ranks * max tokens] records
    uint64_t combine_x[2];
    uint64_t combine_w[2];
    uint64_t combine_flag;     // [2 parities][ranks][flag chunks] uint32 rows-landed counters of the arrival-driven reduce
    int combine_flag_chunks;
    uint64_t end;
};

// `hidden` in elements; the regions are sized for the widest payload (bf16), so an FP8
// and a BF16 dispatch of the same (tokens, hidden, topk) share one partition.
EP_HD HtLayout ht_layout(int num_ranks, int num_max_tokens, int hidden, int num_topk) {
    HtLayout l;
    const uint64_t rows = static_cast<uint64_t>(num_ranks) * num_max_tokens;
    const uint64_t rec_bytes = align_up<uint64_t>(rows * align_up<uint64_t>(hidden * 2 + ht_meta_bytes_max(hidden, num_topk), 128), 256);
    const int lanes = num_ranks > num_topk ? num_ranks : num_topk;   // rank layout or top-k layout
    const uint64_t crow = align_up<uint64_t>(static_cast<uint64_t>(lanes) * num_max_tokens * hidden * 2, 256);
    const uint64_t cw = align_up<uint64_t>(static_cast<uint64_t>(lanes) * num_max_tokens * num_topk * 4, 256);
    uint64_t off = kCtlBytes;
    for (int s = 0; s < 2; ++s) { l.dispatch_rec[s] = off; off += rec_bytes; }
    for (int s = 0; s < 2; ++s) { l.combine_x[s] = off; off += crow; l.combine_w[s] = off; off += cw; }
    l.combine_flag_chunks = static_cast<int>(ceil_div<uint64_t>(rows, kCombineFlagRows));
    l.combine_flag = off;
    off += align_up<uint64_t>(2ull * num_ranks * l.combine_flag_chunks * 4, 256);
    l.end = align_up<uint64_t>(off, kHeapAlignment);
    return l;
}

// ---------------------------------------------------------------- low-latency EP layout
// Two halves (calls alternate). Per half:
//   recv_x        [local experts][ranks][max tokens] messages: 16-byte header whose first word is
//                 (call number << 32 | top-k lane << 16 | token), written last = the arrival flag;
//                 payload (e4m3 + 1x128 scales, or bf16)
//   recv_count    [local experts][ranks] epoch-tagged words (count of the messages above)
//   combine_x     [kMaxLLTopk][max tokens] bf16 rows, indexed by the token's top-k lane
//   combine_flag  [kMaxLLTopk][max tokens] call-tagged words ("the row of this (lane, token) has landed")
//   send_x        [local experts][ranks * max tokens] bf16 rows: optional staging area the caller may
//                 let its expert GEMM write into (zero-copy combine)
constexpr int kMaxLLTopk = 16;

EP_HD int ll_dispatch_msg_bytes(int hidden, bool fp8) {
    const int payload = fp8 ? hidden + align_up(ceil_div(hidden, 128) * 4, 16) : hidden * 2;
    return 16 + payload;
}

struct LLLayout {
    uint64_t recv_x[2];
    uint64_t recv_count[2];
    uint64_t combine_x[2];
    uint64_t combine_flag[2];
    uint64_t send_x[2];
    uint64_t end;
};

// Bytes of one [lane][token] slot of the combine area. A LogFMT row is a table of (amax, amin) bf16 pairs, one per
// 128 channels, followed by the groups back to back: 160 bytes for a group in the 10-bit log format, 256 for one
// left in bf16. The slot is sized for the worst case (no group cast).
EP_HD int ll_logfmt_meta_bytes(int hidden) { return align_up(hidden / 128 * 4, 16); }
EP_HD int ll_combine_slot_bytes(int hidden, bool logfmt) { return hidden * 2 + (logfmt ? ll_logfmt_meta_bytes(hidden) : 0); }

EP_HD LLLayout ll_layout(int num_ranks, int num_max_tokens, int hidden, int num_experts) {
    LLLayout l;
    const int num_local = num_experts / num_ranks;
    const uint64_t msg = ll_dispatch_msg_bytes(hidden, false);   // widest message
    const uint64_t recv = align_up<uint64_t>(static_cast<uint64_t>(num_local) * num_ranks * num_max_tokens * msg, 256);
    const uint64_t cnt = align_up<uint64_t>(static_cast<uint64_t>(num_local) * num_ranks * 8, 256);
    const uint64_t comb = align_up<uint64_t>(static_cast<uint64_t>(kMaxLLTopk) * num_max_tokens * ll_combine_slot_bytes(hidden, true), 256);
    const uint64_t flag = align_up<uint64_t>(static_cast<uint64_t>(kMaxLLTopk) * num_max_tokens * 8, 256);
    const uint64_t send = align_up<uint64_t>(static_cast<uint64_t>(num_local) * num_ranks * num_max_tokens * hidden * 2, 256);
    uint64_t off = kCtlBytes;
    for (int s = 0; s < 2; ++s) {
        l.recv_x[s] = off; off += recv;
        l.recv_count[s] = off; off += cnt;
        l.combine_x[s] = off; off += comb;
        l.combine_flag[s] = off; off += flag;
        l.send_x[s] = off; off += send;
    }
    l.end = align_up<uint64_t>(off, kHeapAlignment);
    return l;
}

}  // namespace ep
