// Error plumbing shared by the engine, the operator entry points and the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <sstream>
#include <stdexcept>
#include <string>

#include "../../include/kge_b200.h"

namespace kge {

// Carries the status code of include/kge_b200.h together with the message.
struct Error : std::exception {
    int code;
    std::string message;
    Error(int code, std::string message) : code(code), message(std::move(message)) {}
    const char* what() const noexcept override { return message.c_str(); }
};

[[noreturn]] inline void fail(int code, const std::string& message) { throw Error(code, message); }

// Streams pieces into a message: msg() << "a" << 3.
struct msg {
    std::ostringstream os;
    template <class T>
    msg& operator<<(const T& v) {
        os << v;
        return *this;
    }
    operator std::string() const { return os.str(); }
};

inline void cuda_check(cudaError_t err, const char* what, const char* file, int line) {
    if (err != cudaSuccess) {
        fail(KGE_DEVICE_STATUS, msg() << "CUDA error in " << what << " at " << file << ":" << line
                                      << ": " << cudaGetErrorString(err));
    }
}
#define KGE_CUDA(call) ::kge::cuda_check((call), #call, __FILE__, __LINE__)

inline size_t round_up(size_t v, size_t to) { return (v + to - 1) / to * to; }

}  // namespace kge
