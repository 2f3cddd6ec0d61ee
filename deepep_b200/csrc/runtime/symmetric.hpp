// Symmetric heap of one rank: a device allocation that every peer of the NVLink domain maps
// into its own address space, so that kernels reach a peer's memory with plain loads, stores
// and bulk copies at heap[peer] + offset.
//
// Two allocators behind one interface:
//   * kIpc  `cudaMalloc`, exported as a CUDA IPC handle (the default);
//   * kVmm  CUDA virtual memory management (EP_HEAP_BACKEND=vmm): ONE reserved address range per
//           rank holds the GPU segment (`cuMemCreate` on the device) and, right behind it, an
//           optional pinned CPU segment on the GPU's NUMA node (`cuMemCreate` with a host-NUMA
//           location), so device code addresses both through the same base pointer. Both
//           allocations are exported as POSIX file descriptors; the descriptors travel between
//           the processes of the box over an abstract unix socket (SCM_RIGHTS), and every peer
//           maps them into a range of its own in the same order.
// Three ways to build the peer table:
//   * processes (one per GPU), IPC: the handles travel over the torch process group;
//   * processes, VMM: the socket names travel over the process group, the descriptors over the sockets;
//   * one process holding several heaps on one device (single-GPU emulation of a multi-rank
//     job, used by the tests): the raw pointers are shared directly.
//
// Parity: csrc/kernels/backend/symmetric.hpp (GPUSymmetricMemory, ElasticSymmetricMemory :145-186,
// HybridElasticSymmetricMemory :191-289: address reserve / create / map / set-access, POSIX-FD import)
// and csrc/utils/shared_memory.hpp:10-125 (SharedMemoryAllocator, IPC path) of the reference, plus the
// pointer-table role of NCCLSymmetricMemoryContext::get_sym_ptr (csrc/kernels/backend/nccl.cu:150-163).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../common/exception.hpp"
#include "../common/layout.hpp"

namespace ep {

// ------------------------------------------------------------------------ driver entry points (no link against libcuda)
struct VmmDriver {
    CUresult (*mem_create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*mem_release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*address_reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*mem_map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*mem_unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    bool ok = false;

    static const VmmDriver& get() {
        static const VmmDriver d = load();
        return d;
    }

private:
    template <typename Fn>
    static bool sym(const char* name, Fn& fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess || p == nullptr) return false;
        fn = reinterpret_cast<Fn>(p);
        return true;
    }
    static VmmDriver load() {
        VmmDriver d;
        d.ok = sym("cuMemCreate", d.mem_create) && sym("cuMemRelease", d.mem_release) && sym("cuMemAddressReserve", d.address_reserve) &&
               sym("cuMemAddressFree", d.address_free) && sym("cuMemMap", d.mem_map) && sym("cuMemUnmap", d.mem_unmap) &&
               sym("cuMemSetAccess", d.set_access) && sym("cuMemExportToShareableHandle", d.export_handle) &&
               sym("cuMemImportFromShareableHandle", d.import_handle) && sym("cuMemGetAllocationGranularity", d.granularity);
        return d;
    }
};

#define EP_DRIVER_CHECK(expr)                                                                           \
    do {                                                                                                \
        const CUresult ep_driver_rc = (expr);                                                           \
        if (ep_driver_rc != CUDA_SUCCESS)                                                               \
            throw ::ep::EPException("CUDA driver", __FILE__, __LINE__, std::string(#expr) + " failed with code " + std::to_string(static_cast<int>(ep_driver_rc))); \
    } while (0)

// ------------------------------------------------------------------------ descriptor passing between the processes of one box
namespace fdpass {

inline sockaddr_un abstract_addr(const std::string& name, socklen_t* len) {
    sockaddr_un a;
    std::memset(&a, 0, sizeof(a));
    a.sun_family = AF_UNIX;
    const size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
    std::memcpy(a.sun_path + 1, name.data(), n);                 // leading NUL = abstract namespace, nothing to unlink
    *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
    return a;
}

inline bool send_fds(int sock, const int* fds, int n) {
    char payload = 'F';
    iovec iov{&payload, 1};
    char control[CMSG_SPACE(sizeof(int) * 4)];
    std::memset(control, 0, sizeof(control));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * n);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * n);
    std::memcpy(CMSG_DATA(c), fds, sizeof(int) * n);
    return sendmsg(sock, &msg, 0) == 1;
}

inline bool recv_fds(int sock, int* fds, int n) {
    char payload = 0;
    iovec iov{&payload, 1};
    char control[CMSG_SPACE(sizeof(int) * 4)];
    std::memset(control, 0, sizeof(control));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = CMSG_SPACE(sizeof(int) * n);
    if (recvmsg(sock, &msg, 0) != 1) return false;
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS || c->cmsg_len != CMSG_LEN(sizeof(int) * n)) return false;
    std::memcpy(fds, CMSG_DATA(c), sizeof(int) * n);
    return true;
}

}  // namespace fdpass

class SymmetricHeap {
public:
    enum class Backend { kIpc, kVmm };

    static Backend backend_from_env() {
        const char* v = std::getenv("EP_HEAP_BACKEND");
        return (v != nullptr && std::string(v) == "vmm") ? Backend::kVmm : Backend::kIpc;
    }

    // `num_cpu_bytes` > 0 (VMM only): a pinned CPU segment follows the GPU segment in the same address range.
    SymmetricHeap(int rank, int num_ranks, size_t num_bytes, Backend backend = backend_from_env(), size_t num_cpu_bytes = 0)
        : rank_(rank), num_ranks_(num_ranks), num_bytes_(num_bytes), num_cpu_bytes_(num_cpu_bytes), backend_(backend) {
        EP_HOST_ASSERT(num_ranks >= 1 && num_ranks <= kMaxRanks);
        EP_HOST_ASSERT(rank >= 0 && rank < num_ranks);
        EP_HOST_ASSERT(num_bytes % kHeapAlignment == 0);
        CUDA_RUNTIME_CHECK(cudaGetDevice(&device_));
        peers_.assign(num_ranks, nullptr);
        if (backend_ == Backend::kVmm) {
            EP_HOST_ASSERT_MSG(VmmDriver::get().ok, "the CUDA driver does not offer the virtual memory management entry points");
            allocate_vmm();
        } else {
            EP_HOST_ASSERT_MSG(num_cpu_bytes == 0, "a CPU segment inside the heap needs EP_HEAP_BACKEND=vmm");
            CUDA_RUNTIME_CHECK(cudaMalloc(&base_, num_bytes));
        }
        // control words start at epoch 0, arrival counters that live in the data regions at zero
        CUDA_RUNTIME_CHECK(cudaMemset(base_, 0, num_bytes));
        if (num_cpu_bytes_ > 0) std::memset(static_cast<uint8_t*>(base_) + num_bytes_, 0, num_cpu_bytes_);
        peers_[rank] = static_cast<uint8_t*>(base_);
    }

    ~SymmetricHeap() { release(); }
    SymmetricHeap(const SymmetricHeap&) = delete;
    SymmetricHeap& operator=(const SymmetricHeap&) = delete;

    // What travels over the process group: the IPC handle, or "vmm:<socket name>" (the descriptors follow over that socket).
    std::string export_handle() {
        if (backend_ == Backend::kVmm) {
            if (socket_name_.empty()) start_fd_server();
            return "vmm:" + socket_name_;
        }
        cudaIpcMemHandle_t handle;
        CUDA_RUNTIME_CHECK(cudaIpcGetMemHandle(&handle, base_));
        return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
    }

    // handles[r] = export_handle() of rank r (the own entry is ignored)
    void open_peers(const std::vector<std::string>& handles) {
        EP_HOST_ASSERT(static_cast<int>(handles.size()) == num_ranks_);
        for (int r = 0; r < num_ranks_; ++r) {
            if (r == rank_) continue;
            if (backend_ == Backend::kVmm) {
                EP_HOST_ASSERT_MSG(handles[r].rfind("vmm:", 0) == 0, "all ranks must use the same heap backend");
                peers_[r] = import_vmm(handles[r].substr(4));
            } else {
                EP_HOST_ASSERT(handles[r].size() == sizeof(cudaIpcMemHandle_t));
                cudaIpcMemHandle_t handle;
                std::memcpy(&handle, handles[r].data(), sizeof(handle));
                void* ptr = nullptr;
                CUDA_RUNTIME_CHECK(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess));
                peers_[r] = static_cast<uint8_t*>(ptr);
                opened_.push_back(ptr);
            }
        }
        connected_ = true;
    }

    // All peers have imported this rank's descriptors (the caller has passed a barrier): stop serving them.
    void finish_export() { stop_fd_server(); }

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
        stop_fd_server();
        if (backend_ == Backend::kVmm) {
            const VmmDriver& d = VmmDriver::get();
            for (auto& m : imported_) {
                d.mem_unmap(m.va, m.total);
                for (auto h : m.handles) d.mem_release(h);
                d.address_free(m.va, m.total);
            }
            imported_.clear();
            const size_t total = num_bytes_ + cpu_mapped_bytes_;
            d.mem_unmap(reinterpret_cast<CUdeviceptr>(base_), total);
            d.mem_release(gpu_handle_);
            if (cpu_mapped_bytes_ > 0) d.mem_release(cpu_handle_);
            d.address_free(reinterpret_cast<CUdeviceptr>(base_), total);
            if (gpu_fd_ >= 0) close(gpu_fd_);
            if (cpu_fd_ >= 0) close(cpu_fd_);
            gpu_fd_ = cpu_fd_ = -1;
        } else {
            for (void* p : opened_) cudaIpcCloseMemHandle(p);
            opened_.clear();
            cudaFree(base_);
        }
        base_ = nullptr;
    }

    uint8_t* base() const { return static_cast<uint8_t*>(base_); }
    uint8_t* peer(int r) const { return peers_[r]; }
    size_t num_bytes() const { return num_bytes_; }
    size_t num_cpu_bytes() const { return num_cpu_bytes_; }
    // the CPU segment of rank r as this rank's kernels (and, for the own one, host code) address it
    uint8_t* cpu_segment(int r) const { return num_cpu_bytes_ > 0 && peers_[r] != nullptr ? peers_[r] + num_bytes_ : nullptr; }
    bool connected() const { return connected_ || num_ranks_ == 1; }
    int device() const { return device_; }
    Backend backend() const { return backend_; }

private:
    struct Imported {
        CUdeviceptr va;
        size_t total;
        std::vector<CUmemGenericAllocationHandle> handles;
    };

    CUmemAccessDesc access_desc() const {
        CUmemAccessDesc a{};
        a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        a.location.id = device_;
        a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        return a;
    }

    void allocate_vmm() {
        const VmmDriver& d = VmmDriver::get();
        CUmemAllocationProp prop{};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = device_;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t gran = 0;
        EP_DRIVER_CHECK(d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
        EP_HOST_ASSERT_MSG(kHeapAlignment % gran == 0 || gran % kHeapAlignment == 0, "unexpected allocation granularity");
        EP_HOST_ASSERT_MSG(num_bytes_ % gran == 0, "heap size must be a multiple of the allocation granularity");
        cpu_mapped_bytes_ = 0;
        CUmemAllocationProp host_prop{};
        if (num_cpu_bytes_ > 0) {
            host_prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
            host_prop.location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
            int numa = 0;
            cudaDeviceGetAttribute(&numa, cudaDevAttrHostNumaId, device_);
            host_prop.location.id = numa < 0 ? 0 : numa;
            host_prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            size_t host_gran = 0;
            EP_DRIVER_CHECK(d.granularity(&host_gran, &host_prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
            cpu_mapped_bytes_ = align_up<size_t>(num_cpu_bytes_, std::max(host_gran, gran));
        }
        const size_t total = num_bytes_ + cpu_mapped_bytes_;
        CUdeviceptr va = 0;
        EP_DRIVER_CHECK(d.address_reserve(&va, total, kHeapAlignment, 0, 0));
        EP_DRIVER_CHECK(d.mem_create(&gpu_handle_, num_bytes_, &prop, 0));
        EP_DRIVER_CHECK(d.mem_map(va, num_bytes_, 0, gpu_handle_, 0));
        if (cpu_mapped_bytes_ > 0) {
            EP_DRIVER_CHECK(d.mem_create(&cpu_handle_, cpu_mapped_bytes_, &host_prop, 0));
            EP_DRIVER_CHECK(d.mem_map(va + num_bytes_, cpu_mapped_bytes_, 0, cpu_handle_, 0));
        }
        std::vector<CUmemAccessDesc> acc{access_desc()};
        if (cpu_mapped_bytes_ > 0) {
            // the own CPU segment is also touched by host code
            CUmemAccessDesc host{};
            host.location = host_prop.location;
            host.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
            EP_DRIVER_CHECK(d.set_access(va, num_bytes_, acc.data(), 1));
            acc.push_back(host);
            EP_DRIVER_CHECK(d.set_access(va + num_bytes_, cpu_mapped_bytes_, acc.data(), acc.size()));
        } else {
            EP_DRIVER_CHECK(d.set_access(va, total, acc.data(), 1));
        }
        EP_DRIVER_CHECK(d.export_handle(&gpu_fd_, gpu_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        if (cpu_mapped_bytes_ > 0) EP_DRIVER_CHECK(d.export_handle(&cpu_fd_, cpu_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        base_ = reinterpret_cast<void*>(va);
    }

    // ---- serving the descriptors: one accept loop on an abstract unix socket until finish_export()
    void start_fd_server() {
        static std::atomic<int> counter{0};
        socket_name_ = "deepep_b200_heap_" + std::to_string(getpid()) + "_" + std::to_string(counter.fetch_add(1)) + "_" + std::to_string(rank_);
        server_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        EP_HOST_ASSERT_MSG(server_fd_ >= 0, "cannot create the unix socket that hands out the heap's descriptors");
        socklen_t len = 0;
        const sockaddr_un addr = fdpass::abstract_addr(socket_name_, &len);
        EP_HOST_ASSERT_MSG(bind(server_fd_, reinterpret_cast<const sockaddr*>(&addr), len) == 0 && listen(server_fd_, kMaxRanks) == 0,
                           "cannot listen on the unix socket that hands out the heap's descriptors");
        stop_server_ = false;
        server_ = std::thread([this]() {
            while (!stop_server_) {
                timeval tv{0, 100000};
                fd_set set;
                FD_ZERO(&set);
                FD_SET(server_fd_, &set);
                if (select(server_fd_ + 1, &set, nullptr, nullptr, &tv) <= 0) continue;
                const int conn = accept(server_fd_, nullptr, nullptr);
                if (conn < 0) continue;
                int fds[2] = {gpu_fd_, cpu_fd_};
                fdpass::send_fds(conn, fds, cpu_fd_ >= 0 ? 2 : 1);
                close(conn);
            }
        });
    }

    void stop_fd_server() {
        if (!server_.joinable()) return;
        stop_server_ = true;
        server_.join();
        close(server_fd_);
        server_fd_ = -1;
    }

    uint8_t* import_vmm(const std::string& name) {
        const VmmDriver& d = VmmDriver::get();
        int sock = -1;
        socklen_t len = 0;
        const sockaddr_un addr = fdpass::abstract_addr(name, &len);
        bool connected = false;
        for (int attempt = 0; attempt < 200 && !connected; ++attempt) {       // the peer may not be listening yet
            sock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
            EP_HOST_ASSERT(sock >= 0);
            connected = connect(sock, reinterpret_cast<const sockaddr*>(&addr), len) == 0;
            if (!connected) {
                close(sock);
                usleep(50000);
            }
        }
        EP_HOST_ASSERT_MSG(connected, "cannot reach a peer's descriptor socket (are all ranks on one machine?)");
        const int n = num_cpu_bytes_ > 0 ? 2 : 1;
        int fds[2] = {-1, -1};
        const bool got = fdpass::recv_fds(sock, fds, n);
        close(sock);
        EP_HOST_ASSERT_MSG(got, "a peer did not hand over its heap descriptors");
        Imported m;
        m.total = num_bytes_ + cpu_mapped_bytes_;
        EP_DRIVER_CHECK(d.address_reserve(&m.va, m.total, kHeapAlignment, 0, 0));
        CUmemGenericAllocationHandle h = 0;
        EP_DRIVER_CHECK(d.import_handle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[0])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
        EP_DRIVER_CHECK(d.mem_map(m.va, num_bytes_, 0, h, 0));
        m.handles.push_back(h);
        if (n == 2) {
            EP_DRIVER_CHECK(d.import_handle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[1])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
            EP_DRIVER_CHECK(d.mem_map(m.va + num_bytes_, cpu_mapped_bytes_, 0, h, 0));
            m.handles.push_back(h);
        }
        const CUmemAccessDesc acc = access_desc();
        EP_DRIVER_CHECK(d.set_access(m.va, m.total, &acc, 1));
        close(fds[0]);
        if (n == 2) close(fds[1]);
        imported_.push_back(m);
        return reinterpret_cast<uint8_t*>(m.va);
    }

    int rank_, num_ranks_;
    size_t num_bytes_, num_cpu_bytes_;
    Backend backend_;
    int device_ = 0;
    void* base_ = nullptr;
    std::vector<uint8_t*> peers_;
    std::vector<void*> opened_;
    bool connected_ = false;
    // VMM state
    CUmemGenericAllocationHandle gpu_handle_ = 0, cpu_handle_ = 0;
    size_t cpu_mapped_bytes_ = 0;
    int gpu_fd_ = -1, cpu_fd_ = -1;
    std::vector<Imported> imported_;
    std::string socket_name_;
    int server_fd_ = -1;
    std::thread server_;
    std::atomic<bool> stop_server_{false};
};

}  // namespace ep
