// Host-side error types and check macros. Device code never traps: device failures are
// reported through status words (see device_utils.cuh) and surface here as EPTimeoutError.
//
// Parity: deep_ep/include/deep_ep/common/exception.cuh:11-94 of the reference
// (EPException, EP_HOST_ASSERT, CUDA_RUNTIME_CHECK, CUDA_DRIVER_CHECK).
#pragma once

#include <cuda_runtime.h>
#include <exception>
#include <sstream>
#include <string>

namespace ep {

class EPException : public std::exception {
public:
    EPException(const char* kind, const char* file, int line, const std::string& what) {
        std::ostringstream os;
        os << kind << " failed at " << file << ":" << line << ": " << what;
        message_ = os.str();
    }
    const char* what() const noexcept override { return message_.c_str(); }

private:
    std::string message_;
};

// A bounded device or host wait ran out. `record` is the raw status word of the rank.
class EPTimeoutError : public std::exception {
public:
    EPTimeoutError(const std::string& what, unsigned long long record) : message_(what), record_(record) {}
    const char* what() const noexcept override { return message_.c_str(); }
    unsigned long long record() const { return record_; }

private:
    std::string message_;
    unsigned long long record_;
};

}  // namespace ep

#define EP_HOST_ASSERT(cond)                                                        \
    do {                                                                            \
        if (!(cond)) throw ep::EPException("Assertion", __FILE__, __LINE__, #cond); \
    } while (0)

#define EP_HOST_ASSERT_MSG(cond, msg)                                             \
    do {                                                                          \
        if (!(cond)) throw ep::EPException("Assertion", __FILE__, __LINE__, msg); \
    } while (0)

#define CUDA_RUNTIME_CHECK(expr)                                                                       \
    do {                                                                                               \
        const cudaError_t e_ = (expr);                                                                 \
        if (e_ != cudaSuccess) throw ep::EPException("CUDA runtime", __FILE__, __LINE__, cudaGetErrorString(e_)); \
    } while (0)
