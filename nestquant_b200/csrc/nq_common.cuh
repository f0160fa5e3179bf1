// Host-side helpers shared by the C ABI translation units: error reporting and argument checks.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/nestquant_b200.h"

namespace nq {

// thread-local message of the last failure (read through nq_last_error)
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define NQ_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return ::nq::fail(NQ_ERR_ARG, __VA_ARGS__); \
    } while (0)

// call right after a kernel launch: reports launch-configuration errors without synchronising
inline int check_launch(const char* what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(NQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return NQ_OK;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace nq
