// Host-side helpers shared by the translation units of libi8f: thread-local
// error text, argument checks and the dtype table.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../include/i8f.h"

namespace i8f {

char* error_buffer();  // thread-local, 512 bytes (defined in api.cu)

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int dtype_size(int dt) {
    switch (dt) {
        case I8F_BF16: return 2;
        case I8F_F16: return 2;
        case I8F_F32: return 4;
        default: return 0;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

void count_launch();  // one more kernel launched by the library (defined in api.cu)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(I8F_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    count_launch();
    return I8F_OK;
}

int* device_status_word();  // device address of the status word on the current device, or nullptr

}  // namespace i8f

#define I8F_REQUIRE(cond, code, ...)                    \
    do {                                                \
        if (!(cond)) return ::i8f::fail(code, __VA_ARGS__); \
    } while (0)
