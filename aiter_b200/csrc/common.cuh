// Shared host-side helpers of libaiter_b200.so: error bridging of the C-ABI, tensor checks.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>

#include "../../include/aiter_b200.h"

namespace b200 {

// Thread-local message of the last failed call (same contract as the reference's
// g_aiter_last_error, csrc/include/aiter_ctypes_error.h:61-71). Defined in abi.cu.
std::string& last_error();

template <typename... Args>
[[noreturn]] inline void fail(Args&&... args) {
    std::ostringstream os;
    (os << ... << args);
    throw std::runtime_error(os.str());
}

#define B200_CHECK(cond, ...)                         \
    do {                                              \
        if (!(cond)) ::b200::fail(__VA_ARGS__);       \
    } while (0)

#define B200_CUDA(expr)                                                                   \
    do {                                                                                  \
        cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess)                                                            \
            ::b200::fail(#expr, " failed: ", cudaGetErrorName(e_), " (", cudaGetErrorString(e_), ")"); \
    } while (0)

// Runs fn, converts any C++ exception into status -1 + thread-local message; exceptions never
// cross the C boundary.
template <typename Fn>
inline int safe_call(Fn&& fn) {
    last_error().clear();
    try {
        fn();
        return 0;
    } catch (const std::exception& e) {
        last_error() = e.what();
        return -1;
    } catch (...) {
        last_error() = "unknown C++ exception";
        return -1;
    }
}

inline bool is_contiguous(const aiter_tensor_t* t) {
    if (t->numel_ == 0) return true;
    int64_t expected = 1;
    for (int d = t->ndim - 1; d >= 0; --d) {
        if (t->shape[d] != 1 && t->strides[d] != expected) return false;
        expected *= t->shape[d];
    }
    return true;
}

inline void check_tensor(const aiter_tensor_t* t, const char* name, int dtype, int ndim) {
    B200_CHECK(t != nullptr, name, " must not be NULL");
    B200_CHECK(t->ndim >= 0 && t->ndim <= 8, name, ": bad ndim ", t->ndim);
    B200_CHECK(t->device_id >= 0, name, " must be a CUDA tensor");
    B200_CHECK(dtype < 0 || t->dtype_ == dtype, name, ": unexpected dtype code ", t->dtype_,
               " (want ", dtype, ")");
    B200_CHECK(ndim < 0 || t->ndim == ndim, name, ": expected ", ndim, " dims, got ", t->ndim);
    B200_CHECK(is_contiguous(t), name, " must be contiguous");
    B200_CHECK(t->numel_ == 0 || t->ptr != nullptr, name, ": NULL data pointer");
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        B200_CUDA(cudaGetDevice(&prev));
        if (prev != dev) B200_CUDA(cudaSetDevice(dev));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

inline int sm_count(int dev) {
    static int cached[64] = {0};
    if (dev < 64 && cached[dev] > 0) return cached[dev];
    int n = 0;
    B200_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 64) cached[dev] = n;
    return n;
}

}  // namespace b200
