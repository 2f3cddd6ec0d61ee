// CPU segment of a rank: pinned host memory that the rank's own GPU and the GPUs of the other
// processes on the machine can read with ordinary loads (over PCIe), used for tables that are too
// large or too cold for device memory (Engram storage with `num_cpu_bytes`).
//
// The memory is a POSIX shared-memory object mapped into every process that opens it and registered
// with CUDA there (cudaHostRegisterMapped | cudaHostRegisterPortable), so each process gets its own
// device-visible address of the same pages. The creating process unlinks the name when it closes
// the segment; mappings that are still open stay valid until they are unmapped.
//
// Pages are placed by the kernel's first-touch policy: create the segment from a thread that runs on
// the NUMA node of the GPU (deepep_b200.utils.numa.bind_to_gpu_node) to keep it next to that GPU.
//
// Parity: ElasticSymmetricMemory / HybridElasticSymmetricMemory of the reference
// (csrc/kernels/backend/symmetric.hpp: a NUMA-local host segment inside the symmetric window, shared
// through POSIX file descriptors). With the cudaMalloc / IPC heap the host segment is this separate mapping;
// with the virtual-memory heap (EP_HEAP_BACKEND=vmm) it is part of the heap's own address range, right behind
// the GPU segment, and `window()` only wraps those addresses.
#pragma once

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <memory>
#include <random>
#include <string>

#include "../common/exception.hpp"

namespace ep {

class HostSegment {
public:
    static std::shared_ptr<HostSegment> create(size_t num_bytes) {
        static std::atomic<int> counter{0};
        std::random_device rd;
        const std::string name = "/deepep_b200_" + std::to_string(getpid()) + "_" + std::to_string(counter++) + "_" + std::to_string(rd());
        const int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
        EP_HOST_ASSERT_MSG(fd >= 0, "shm_open failed for a new host segment");
        if (ftruncate(fd, static_cast<off_t>(num_bytes)) != 0) {
            close(fd);
            shm_unlink(name.c_str());
            EP_HOST_ASSERT_MSG(false, "cannot size the host segment (is /dev/shm large enough?)");
        }
        return std::shared_ptr<HostSegment>(new HostSegment(name, num_bytes, fd, true));
    }

    // A CPU segment that lives inside a symmetric heap's address range (nothing is owned here): `device` is the
    // address kernels of this process use, `host` the address host code may use (null for a peer's segment).
    static std::shared_ptr<HostSegment> window(uint8_t* device, uint8_t* host, size_t num_bytes) {
        auto s = std::shared_ptr<HostSegment>(new HostSegment());
        s->name_ = "(heap window)";
        s->num_bytes_ = num_bytes;
        s->device_ = device;
        s->host_ = host;
        s->window_ = true;
        return s;
    }

    static std::shared_ptr<HostSegment> open(const std::string& name, size_t num_bytes) {
        const int fd = shm_open(name.c_str(), O_RDWR, 0600);
        EP_HOST_ASSERT_MSG(fd >= 0, "shm_open failed for a peer's host segment");
        return std::shared_ptr<HostSegment>(new HostSegment(name, num_bytes, fd, false));
    }

    ~HostSegment() { release(); }
    HostSegment(const HostSegment&) = delete;
    HostSegment& operator=(const HostSegment&) = delete;

    void release() {
        if (window_) {
            host_ = device_ = nullptr;
            return;
        }
        if (host_ == nullptr) return;
        cudaHostUnregister(host_);
        munmap(host_, num_bytes_);
        host_ = nullptr;
        device_ = nullptr;
        if (owner_) shm_unlink(name_.c_str());
    }

    const std::string& name() const { return name_; }
    size_t num_bytes() const { return num_bytes_; }
    uint8_t* host_ptr() const { return static_cast<uint8_t*>(host_); }
    uint8_t* device_ptr() const { return static_cast<uint8_t*>(device_); }   // address of the pages as seen by kernels of this process

private:
    HostSegment() : num_bytes_(0), owner_(false) {}
    HostSegment(std::string name, size_t num_bytes, int fd, bool owner) : name_(std::move(name)), num_bytes_(num_bytes), owner_(owner) {
        host_ = mmap(nullptr, num_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (host_ == MAP_FAILED) {
            host_ = nullptr;
            if (owner) shm_unlink(name_.c_str());
            EP_HOST_ASSERT_MSG(false, "mmap of the host segment failed");
        }
        if (owner) std::memset(host_, 0, num_bytes);     // first touch: the pages land on this thread's NUMA node
        if (cudaHostRegister(host_, num_bytes, cudaHostRegisterMapped | cudaHostRegisterPortable) != cudaSuccess ||
            cudaHostGetDevicePointer(&device_, host_, 0) != cudaSuccess) {
            cudaGetLastError();
            munmap(host_, num_bytes);
            host_ = nullptr;
            if (owner) shm_unlink(name_.c_str());
            EP_HOST_ASSERT_MSG(false, "cannot register the host segment with CUDA");
        }
    }

    std::string name_;
    size_t num_bytes_;
    bool owner_;
    bool window_ = false;
    void* host_ = nullptr;
    void* device_ = nullptr;
};

}  // namespace ep
