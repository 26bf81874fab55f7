// Shared host-side helpers of libkhcuda_gqa: status codes, the thread-local error message and
// checked integer arithmetic. Nothing here touches the GPU.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/kh_gqa.h"

namespace kh {

// Records `message` for kh_last_error() on the calling thread and returns `code`.
kh_status fail(kh_status code, const char* format, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
const std::string& last_error();

// Thrown by the internal host logic where the reference would panic; converted into a status
// code and message at the C boundary so nothing unwinds across it.
struct Failure {
    kh_status code;
    std::string message;
};

[[noreturn]] void raise(kh_status code, const char* format, ...) __attribute__((format(printf, 2, 3)));

#define KH_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) ::kh::raise(KH_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

// Runs `body` (a lambda returning kh_status) and maps a Failure to its status code.
template <typename F>
kh_status guarded(F&& body) {
    try {
        clear_error();
        return body();
    } catch (const Failure& failure) {
        return fail(failure.code, "%s", failure.message.c_str());
    } catch (const std::exception& error) {
        return fail(KH_INTERNAL, "%s", error.what());
    }
}

inline uint64_t mul_u64(uint64_t a, uint64_t b, const char* what) {
    uint64_t r;
    if (__builtin_mul_overflow(a, b, &r)) raise(KH_INVALID_ARGUMENT, "%s must fit u64", what);
    return r;
}

inline uint32_t to_u32(uint64_t value, const char* what) {
    if (value > 0xffffffffull) raise(KH_INVALID_ARGUMENT, "%s must fit u32", what);
    return static_cast<uint32_t>(value);
}

inline uint32_t mul_u32(uint32_t a, uint32_t b, const char* what) { return to_u32(uint64_t(a) * uint64_t(b), what); }

inline uint32_t div_ceil(uint32_t a, uint32_t b) { return a / b + (a % b != 0); }
inline uint64_t div_ceil64(uint64_t a, uint64_t b) { return a / b + (a % b != 0); }

inline uint32_t ilog2(uint64_t v) { return 63u - static_cast<uint32_t>(__builtin_clzll(v)); }

inline uint32_t next_pow2(uint32_t v) {
    if (v <= 1) return 1;
    return 1u << (32 - __builtin_clz(v - 1));
}

inline uint32_t dtype_size(kh_dtype dtype) {
    switch (dtype) {
        case KH_DTYPE_FLOAT16:
        case KH_DTYPE_BFLOAT16:
            return 2;
        case KH_DTYPE_FLOAT32:
            return 4;
        case KH_DTYPE_FP8_E4M3FN:
            return 1;
        default:
            return 0;
    }
}

}  // namespace kh
