// Stream-level helpers shared by the host drivers: 64-bit stream memory operations resolved at run time, and a pool
// of side streams for copy-engine transfers that run side by side.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

#include "../common/exception.hpp"

namespace ep {

// ---- stream memory operations (0 SMs): the driver writes / waits for a 64-bit word in stream order
// Parity: csrc/kernels/backend/cuda_driver.cu:12-52 of the reference (batched write / wait-GEQ of AGRS sessions).
// `write` is always used where it is available (a write cannot block). Waits are opt-in (EP_STREAM_MEMOPS=1, `waits`):
// such a wait has no time limit, unlike the wait of a flag kernel, so a peer that never signals blocks the stream
// until the process gives up; the default keeps every wait bounded.
struct StreamMemOps {
    using WriteFn = int (*)(cudaStream_t, unsigned long long, unsigned long long, unsigned int);
    using WaitFn = int (*)(cudaStream_t, unsigned long long, unsigned long long, unsigned int);
    using BatchFn = CUresult (*)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);
    WriteFn write = nullptr;
    WaitFn wait = nullptr;
    BatchFn batch = nullptr;      // several writes / waits in one driver call (optional)
    bool available = false;   // both entry points resolved
    bool waits = false;       // EP_STREAM_MEMOPS=1: flag rounds of AGRS / PP run as stream operations
    StreamMemOps() {
        cudaDriverEntryPointQueryResult res;
        void* w = nullptr;
        void* q = nullptr;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue64", &w, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess) return;
        if (cudaGetDriverEntryPoint("cuStreamWaitValue64", &q, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess) return;
        write = reinterpret_cast<WriteFn>(w);
        wait = reinterpret_cast<WaitFn>(q);
        available = true;
        void* b = nullptr;
        if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &b, cudaEnableDefault, &res) == cudaSuccess && res == cudaDriverEntryPointSuccess)
            batch = reinterpret_cast<BatchFn>(b);
        const char* v = std::getenv("EP_STREAM_MEMOPS");
        waits = v != nullptr && v[0] == '1';
    }
};

inline StreamMemOps& stream_memops() {
    static StreamMemOps ops;
    return ops;
}

// `count` (at most 64) 64-bit writes of `value` to `addrs`, in stream order behind everything queued on `stream`: one
// driver call where the batched form is available, else one call per word
inline void stream_write_values(cudaStream_t stream, const unsigned long long* addrs, int count, unsigned long long value) {
    StreamMemOps& ops = stream_memops();
    EP_HOST_ASSERT(ops.available && count >= 0 && count <= 64);
    if (count == 0) return;
    if (ops.batch != nullptr && count > 1) {
        CUstreamBatchMemOpParams params[64];
        for (int i = 0; i < count; ++i) {
            params[i] = CUstreamBatchMemOpParams{};
            params[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
            params[i].writeValue.address = static_cast<CUdeviceptr>(addrs[i]);
            params[i].writeValue.value64 = value;
            params[i].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT;
        }
        EP_HOST_ASSERT(ops.batch(reinterpret_cast<CUstream>(stream), static_cast<unsigned int>(count), params, 0) == CUDA_SUCCESS);
        return;
    }
    for (int i = 0; i < count; ++i) EP_HOST_ASSERT(ops.write(stream, addrs[i], value, 0) == 0);
}

// ---- side streams: work item i runs on stream i % kFanStreams, forked from and joined to the caller's stream with
// events, so that copies to different peers use different copy engines instead of queueing behind one another
struct FanOut {
    static constexpr int kFanStreams = 7;
    cudaStream_t streams[kFanStreams] = {};
    cudaEvent_t fork_event = nullptr, join_event[kFanStreams] = {};
    bool ready = false;
    void init() {
        if (ready) return;
        for (auto& st : streams) CUDA_RUNTIME_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
        CUDA_RUNTIME_CHECK(cudaEventCreateWithFlags(&fork_event, cudaEventDisableTiming));
        for (auto& ev : join_event) CUDA_RUNTIME_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        ready = true;
    }
    // the first `used` side streams start behind everything queued on `stream` so far
    void fork(cudaStream_t stream, int used) {
        CUDA_RUNTIME_CHECK(cudaEventRecord(fork_event, stream));
        for (int i = 0; i < std::min(used, kFanStreams); ++i) CUDA_RUNTIME_CHECK(cudaStreamWaitEvent(streams[i], fork_event, 0));
    }
    // `stream` continues behind everything queued on the first `used` side streams
    void join(cudaStream_t stream, int used) {
        for (int i = 0; i < std::min(used, kFanStreams); ++i) {
            CUDA_RUNTIME_CHECK(cudaEventRecord(join_event[i], streams[i]));
            CUDA_RUNTIME_CHECK(cudaStreamWaitEvent(stream, join_event[i], 0));
        }
    }
};

inline FanOut& fan_out(int device) {
    static FanOut pools[64];
    EP_HOST_ASSERT(device >= 0 && device < 64);
    pools[device].init();
    return pools[device];
}

}  // namespace ep
