// Symmetric heap of one rank: a device allocation that every peer of the NVLink domain maps
// into its own address space, so that kernels reach a peer's memory with plain loads, stores
// and bulk copies at heap[peer] + offset.
//
// Two ways to build the peer table:
//   * processes (one per GPU): the allocation is exported as a CUDA IPC handle, the handles
//     travel over the torch process group, and every peer opens them;
//   * one process holding several heaps on one device (single-GPU emulation of a multi-rank
//     job, used by the tests): the raw pointers are shared directly.
//
// Parity: csrc/kernels/backend/symmetric.hpp (GPUSymmetricMemory) and
// csrc/utils/shared_memory.hpp:10-125 (SharedMemoryAllocator, IPC path) of the reference,
// plus the pointer-table role of NCCLSymmetricMemoryContext::get_sym_ptr
// (csrc/kernels/backend/nccl.cu:150-163).
#pragma once

#include <cuda_runtime.h>
#include <cstring>
#include <string>
#include <vector>

#include "../common/exception.hpp"
#include "../common/layout.hpp"

namespace ep {

class SymmetricHeap {
public:
    SymmetricHeap(int rank, int num_ranks, size_t num_bytes) : rank_(rank), num_ranks_(num_ranks), num_bytes_(num_bytes) {
        EP_HOST_ASSERT(num_ranks >= 1 && num_ranks <= kMaxRanks);
        EP_HOST_ASSERT(rank >= 0 && rank < num_ranks);
        EP_HOST_ASSERT(num_bytes % kHeapAlignment == 0);
        CUDA_RUNTIME_CHECK(cudaGetDevice(&device_));
        CUDA_RUNTIME_CHECK(cudaMalloc(&base_, num_bytes));
        // control words start at epoch 0, arrival counters that live in the data regions at zero
        CUDA_RUNTIME_CHECK(cudaMemset(base_, 0, num_bytes));
        peers_.assign(num_ranks, nullptr);
        peers_[rank] = static_cast<uint8_t*>(base_);
    }

    ~SymmetricHeap() { release(); }
    SymmetricHeap(const SymmetricHeap&) = delete;
    SymmetricHeap& operator=(const SymmetricHeap&) = delete;

    std::string export_handle() const {
        cudaIpcMemHandle_t handle;
        CUDA_RUNTIME_CHECK(cudaIpcGetMemHandle(&handle, base_));
        return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
    }

    // handles[r] = export_handle() of rank r (the own entry is ignored)
    void open_peers(const std::vector<std::string>& handles) {
        EP_HOST_ASSERT(static_cast<int>(handles.size()) == num_ranks_);
        for (int r = 0; r < num_ranks_; ++r) {
            if (r == rank_) continue;
            EP_HOST_ASSERT(handles[r].size() == sizeof(cudaIpcMemHandle_t));
            cudaIpcMemHandle_t handle;
            std::memcpy(&handle, handles[r].data(), sizeof(handle));
            void* ptr = nullptr;
            CUDA_RUNTIME_CHECK(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess));
            peers_[r] = static_cast<uint8_t*>(ptr);
            opened_.push_back(ptr);
        }
        connected_ = true;
    }

    // same-process peers (single-GPU emulation): share raw pointers
    void set_local_peers(const std::vector<SymmetricHeap*>& heaps) {
        EP_HOST_ASSERT(static_cast<int>(heaps.size()) == num_ranks_);
        for (int r = 0; r < num_ranks_; ++r) {
            EP_HOST_ASSERT(heaps[r]->num_bytes_ == num_bytes_);
            peers_[r] = static_cast<uint8_t*>(heaps[r]->base_);
        }
        connected_ = true;
    }

    void release() {
        if (base_ == nullptr) return;
        for (void* p : opened_) cudaIpcCloseMemHandle(p);
        opened_.clear();
        cudaFree(base_);
        base_ = nullptr;
    }

    uint8_t* base() const { return static_cast<uint8_t*>(base_); }
    uint8_t* peer(int r) const { return peers_[r]; }
    size_t num_bytes() const { return num_bytes_; }
    bool connected() const { return connected_ || num_ranks_ == 1; }
    int device() const { return device_; }

private:
    int rank_, num_ranks_;
    size_t num_bytes_;
    int device_ = 0;
    void* base_ = nullptr;
    std::vector<uint8_t*> peers_;
    std::vector<void*> opened_;
    bool connected_ = false;
};

}  // namespace ep
