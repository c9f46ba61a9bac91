// Helpers shared by the host-side translation units of libmcsparse.so.
//
// Internally every function reports an mcspStatus-like code and the exported wrapper maps
// it to the public status exactly as the reference does
// (mcsparse/src/wrapper/mcsp_interface_wrapper.cpp:5-42):
//   invalid handle            -> MCSPARSE_STATUS_NOT_INITIALIZED
//   invalid pointer/size/value-> MCSPARSE_STATUS_INVALID_VALUE
//   not implemented           -> MCSPARSE_STATUS_NOT_SUPPORTED
//   launch failure            -> MCSPARSE_STATUS_EXECUTION_FAILED
#ifndef MCSPARSE_B200_API_COMMON_H_
#define MCSPARSE_B200_API_COMMON_H_

#include <cstdio>
#include <cstdlib>

#include "internal.h"

namespace mcsp_b200 {
namespace api {

enum St {
    OK = 0,
    BAD_HANDLE,
    BAD_POINTER,
    BAD_SIZE,
    BAD_VALUE,
    NOT_IMPL,
    INTERNAL,
    EXEC_FAILED,
    ALLOC_FAILED,
};

inline mcsparseStatus_t pub(St s) {
    switch (s) {
        case OK: return MCSPARSE_STATUS_SUCCESS;
        case BAD_HANDLE: return MCSPARSE_STATUS_NOT_INITIALIZED;
        case BAD_POINTER:
        case BAD_SIZE:
        case BAD_VALUE: return MCSPARSE_STATUS_INVALID_VALUE;
        case NOT_IMPL: return MCSPARSE_STATUS_NOT_SUPPORTED;
        case EXEC_FAILED: return MCSPARSE_STATUS_EXECUTION_FAILED;
        case ALLOC_FAILED: return MCSPARSE_STATUS_ALLOC_FAILED;
        default: return MCSPARSE_STATUS_INTERNAL_ERROR;
    }
}

inline St from_cuda(cudaError_t e) {
    if (e == cudaSuccess) return OK;
    if (e == cudaErrorMemoryAllocation) return ALLOC_FAILED;
    return EXEC_FAILED;
}

// Warnings go to stderr unless SPARSE_LOG_ENABLE=0, the switch the reference's logger reads
// (mcsparse/src/utils/mcsp_logger.cpp:29-61).
inline void log_error(const char* msg) {
    static const bool enabled = [] {
        const char* v = std::getenv("SPARSE_LOG_ENABLE");
        return !(v && v[0] == '0');
    }();
    if (enabled) std::fprintf(stderr, "[mcsparse] %s\n", msg);
}

inline bool value_type_known(macaDataType t) {
    switch (t) {
        case MACA_R_32F: case MACA_R_64F: case MACA_C_32F: case MACA_C_64F: case MACA_R_16F:
        case MACA_R_16BF: case MACA_C_16F: case MACA_C_16BF: case MACA_R_8I:
            return true;
        default:
            return false;
    }
}

// Makes a device current for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

}  // namespace api
}  // namespace mcsp_b200

#endif  // MCSPARSE_B200_API_COMMON_H_
