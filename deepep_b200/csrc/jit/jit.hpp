// Run-time compilation of specialised kernels: source string -> cubin (nvcc) -> loaded kernel.
//
//   Compiler        builds `name` + `code` with fixed flags into <cache>/kernel.<name>.<digest>/kernel.cubin;
//                   the digest covers the code, the flags, the compiler version and the content of every
//                   library header the code includes (recursively), so editing a header invalidates the
//                   cache. A build happens in a temporary directory that is renamed into place, so
//                   concurrent ranks may race on the same kernel without corrupting the cache.
//   KernelLibrary   loads the cubin with the CUDA runtime library API and looks the kernel up under its
//                   fixed `extern "C"` name (no symbol-table parsing, no disassembly tools).
//   launch          cudaLaunchKernelExC with optional cooperative / cluster attributes; the kernel takes
//                   one parameter block by value, passed as raw bytes.
//
// Parity: csrc/jit/{compiler,kernel_runtime,cache,launch_runtime,include_parser,device_runtime}.hpp of
// the reference. Differences: the kernel name is fixed ("ep_jit_entry") instead of being parsed from
// `cuobjdump -symbols`, and there are no SASS / PTX dump options.
#pragma once

#include <cuda_runtime.h>
#include <sys/stat.h>
#include <unistd.h>

#include <array>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <regex>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "../common/exception.hpp"

namespace ep {
namespace jit {

constexpr const char* kEntryName = "ep_jit_entry";

// ---------------------------------------------------------------- small host utilities
inline std::string get_env(const char* name, const std::string& fallback = "") {
    const char* v = std::getenv(name);
    return v != nullptr ? std::string(v) : fallback;
}

// FNV-1a over the bytes, finished with a splitmix round; 16 hex digits
inline std::string digest(const std::string& data) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : data) {
        h ^= c;
        h *= 1099511628211ull;
    }
    h ^= h >> 30;
    h *= 0xbf58476d1ce4e5b9ull;
    h ^= h >> 27;
    h *= 0x94d049bb133111ebull;
    h ^= h >> 31;
    char buf[17];
    std::snprintf(buf, sizeof(buf), "%016llx", static_cast<unsigned long long>(h));
    return buf;
}

inline std::pair<int, std::string> run_command(const std::string& cmd) {
    std::string out;
    FILE* pipe = popen((cmd + " 2>&1").c_str(), "r");
    if (pipe == nullptr) return {-1, "popen failed"};
    std::array<char, 512> buf;
    while (fgets(buf.data(), buf.size(), pipe) != nullptr) out += buf.data();
    const int rc = pclose(pipe);
    return {rc, out};
}

inline bool file_exists(const std::string& path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0;
}

inline void make_dirs(const std::string& path) {
    std::string cur;
    for (size_t i = 0; i < path.size(); ++i) {
        cur += path[i];
        if (path[i] == '/' || i + 1 == path.size()) mkdir(cur.c_str(), 0755);
    }
}

inline std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

// ---------------------------------------------------------------- include hashing
// Digest of every `#include "..."` header (relative to `include_root`) that `code` pulls in, recursively.
class IncludeParser {
public:
    explicit IncludeParser(std::string include_root) : root_(std::move(include_root)) {}

    std::string hash_of(const std::string& code) {
        std::set<std::string> seen;
        std::string acc;
        collect(code, "", seen, acc);
        return digest(acc);
    }

private:
    void collect(const std::string& code, const std::string& dir, std::set<std::string>& seen, std::string& acc) {
        static const std::regex re("#\\s*include\\s*\"([^\"]+)\"");
        for (auto it = std::sregex_iterator(code.begin(), code.end(), re); it != std::sregex_iterator(); ++it) {
            const std::string rel = (*it)[1];
            std::string path = root_ + "/" + (dir.empty() ? "" : dir + "/") + rel;
            if (!file_exists(path)) path = root_ + "/" + rel;
            if (!file_exists(path) || !seen.insert(path).second) continue;
            const std::string content = read_file(path);
            acc += path + "\n" + content;
            const size_t slash = rel.rfind('/');
            std::string sub = dir;
            if (slash != std::string::npos) sub = (dir.empty() ? "" : dir + "/") + rel.substr(0, slash);
            collect(content, sub, seen, acc);
        }
    }
    std::string root_;
};

// ---------------------------------------------------------------- compiler
class Compiler {
public:
    Compiler(std::string cache_dir, std::string cuda_home, std::string include_root)
        : cache_dir_(std::move(cache_dir)), include_root_(std::move(include_root)), parser_(include_root_) {
        nvcc_ = get_env("EP_JIT_NVCC_COMPILER", cuda_home + "/bin/nvcc");
        flags_ = "-std=c++" + get_env("EP_JIT_CPP_STANDARD", "17") +
                 " -gencode arch=compute_100a,code=sm_100a -O3 --expt-relaxed-constexpr -cubin -I" + include_root_;
        if (get_env("EP_JIT_WITH_LINEINFO") == "1") flags_ += " -lineinfo";
        if (get_env("EP_JIT_PTXAS_VERBOSE") == "1" || get_env("EP_JIT_PTXAS_CHECK") == "1") flags_ += " -Xptxas -v";
        make_dirs(cache_dir_);
    }

    const std::string& flags() const { return flags_; }
    int num_compilations() const { return num_compilations_; }

    std::string version() {
        if (version_.empty()) {
            auto [rc, out] = run_command(nvcc_ + " --version");
            EP_HOST_ASSERT_MSG(rc == 0, "cannot run nvcc for run-time compilation");
            version_ = digest(out);
        }
        return version_;
    }

    // Returns the path of the cubin of (name, code); compiles when the cache has none.
    std::string build(const std::string& name, const std::string& code) {
        const std::string key = digest(name + "\n" + flags_ + "\n" + version() + "\n" + parser_.hash_of(code) + "\n" + code);
        const std::string dir = cache_dir_ + "/kernel." + name + "." + key;
        const std::string cubin = dir + "/kernel.cubin";
        if (file_exists(cubin)) return cubin;
        // build in a private directory, then publish it with an atomic rename (losing a race is fine)
        char host[64] = {0};
        gethostname(host, sizeof(host) - 1);
        const std::string tmp = cache_dir_ + "/tmp." + name + "." + key + "." + host + "." + std::to_string(getpid());
        make_dirs(tmp);
        {
            std::ofstream f(tmp + "/kernel.cu");
            f << code;
        }
        const std::string cmd = nvcc_ + " " + flags_ + " " + tmp + "/kernel.cu -o " + tmp + "/kernel.cubin";
        if (get_env("EP_JIT_PRINT_COMPILER_COMMAND") == "1" || get_env("EP_JIT_DEBUG") == "1") std::printf("[ep jit] %s\n", cmd.c_str());
        auto [rc, out] = run_command(cmd);
        ++num_compilations_;
        if (rc != 0) {
            run_command("rm -rf '" + tmp + "'");
            throw EPException("JIT compilation", __FILE__, __LINE__, name + ":\n" + out);
        }
        if (get_env("EP_JIT_PTXAS_VERBOSE") == "1") std::printf("%s", out.c_str());
        if (get_env("EP_JIT_PTXAS_CHECK") == "1" && std::regex_search(out, std::regex("[1-9][0-9]* bytes spill"))) {
            run_command("rm -rf '" + tmp + "'");
            throw EPException("JIT register check", __FILE__, __LINE__, name + " spills registers:\n" + out);
        }
        if (std::rename(tmp.c_str(), dir.c_str()) != 0) run_command("rm -rf '" + tmp + "'");   // another rank published it first
        EP_HOST_ASSERT_MSG(file_exists(cubin), "JIT cache entry is missing after the build");
        return cubin;
    }

private:
    std::string cache_dir_, include_root_, nvcc_, flags_, version_;
    IncludeParser parser_;
    int num_compilations_ = 0;
};

// ---------------------------------------------------------------- loaded kernels
class KernelLibrary {
public:
    explicit KernelLibrary(const std::string& cubin_path) {
        CUDA_RUNTIME_CHECK(cudaLibraryLoadFromFile(&library_, cubin_path.c_str(), nullptr, nullptr, 0, nullptr, nullptr, 0));
        CUDA_RUNTIME_CHECK(cudaLibraryGetKernel(&kernel_, library_, kEntryName));
    }
    ~KernelLibrary() {
        if (library_ != nullptr) cudaLibraryUnload(library_);
    }
    KernelLibrary(const KernelLibrary&) = delete;
    KernelLibrary& operator=(const KernelLibrary&) = delete;

    // `params` is the kernel's single by-value parameter block
    void launch(dim3 grid, dim3 block, int smem_bytes, cudaStream_t stream, const void* params, bool cooperative, int cluster_dim) const {
        if (smem_bytes > 48 * 1024)
            CUDA_RUNTIME_CHECK(cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel_), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
        cfg.stream = stream;
        cudaLaunchAttribute attrs[2];
        int n = 0;
        if (cooperative) {
            attrs[n].id = cudaLaunchAttributeCooperative;
            attrs[n].val.cooperative = 1;
            ++n;
        }
        if (cluster_dim > 1) {
            attrs[n].id = cudaLaunchAttributeClusterDimension;
            attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster_dim);
            attrs[n].val.clusterDim.y = 1;
            attrs[n].val.clusterDim.z = 1;
            ++n;
        }
        cfg.attrs = attrs;
        cfg.numAttrs = static_cast<unsigned>(n);
        void* args[] = {const_cast<void*>(params)};
        CUDA_RUNTIME_CHECK(cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kernel_), args));
    }

private:
    cudaLibrary_t library_ = nullptr;
    cudaKernel_t kernel_ = nullptr;
};

// in-process cache: cubin path -> loaded library
class KernelCache {
public:
    std::shared_ptr<KernelLibrary> get(const std::string& cubin_path) {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = loaded_.find(cubin_path);
        if (it != loaded_.end()) return it->second;
        auto lib = std::make_shared<KernelLibrary>(cubin_path);
        loaded_[cubin_path] = lib;
        return lib;
    }
    void clear() {
        std::lock_guard<std::mutex> lock(mutex_);
        loaded_.clear();
    }

private:
    std::mutex mutex_;
    std::map<std::string, std::shared_ptr<KernelLibrary>> loaded_;
};

}  // namespace jit
}  // namespace ep
