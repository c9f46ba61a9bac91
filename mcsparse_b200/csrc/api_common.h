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
#include <mutex>
#include <string>

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

// The three switches of the reference's logger (mcsparse/src/utils/mcsp_logger.cpp:29-61):
//   SPARSE_LOG_ENABLE=0   nothing is logged
//   SPARSE_LOG_LEVEL=n    messages above level n are dropped (0 fatal, 1 error, 2 warning, 3 info, 4 debug; default 3)
//   SPARSE_LOG_OUTPUT     "stdout", "file" (mcsparse.txt in the working directory, the reference's fixed name) or
//                         "syslog" (the reference formats nothing for it either); unset: stderr here, where the
//                         reference defaults to stdout, so that a caller's own standard output stays clean.
inline void log_message(int level, const char* msg) {
    struct Cfg {
        bool enabled = true;
        int level = 3;
        int output = 0;  // 0 stderr, 1 stdout, 2 file, 3 syslog
        std::FILE* file = nullptr;
    };
    static Cfg cfg = [] {
        Cfg c;
        if (const char* v = std::getenv("SPARSE_LOG_ENABLE")) c.enabled = std::strtol(v, nullptr, 10) != 0;
        if (const char* v = std::getenv("SPARSE_LOG_LEVEL")) {
            c.level = (int)std::strtol(v, nullptr, 10);
            if (c.level > 4) c.level = 4;
        }
        if (const char* v = std::getenv("SPARSE_LOG_OUTPUT")) {
            const std::string o(v);
            c.output = o == "stdout" ? 1 : o == "file" ? 2 : o == "syslog" ? 3 : 0;
        }
        return c;
    }();
    static std::mutex lock;
    if (!cfg.enabled || level > cfg.level || cfg.output == 3) return;
    static const char* const names[] = {"FATAL", "ERROR", "WARNING", "INFO", "DEBUG"};
    std::lock_guard<std::mutex> g(lock);
    std::FILE* out = cfg.output == 1 ? stdout : stderr;
    if (cfg.output == 2) {
        if (cfg.file == nullptr) cfg.file = std::fopen("mcsparse.txt", "w");
        if (cfg.file != nullptr) out = cfg.file;
    }
    std::fprintf(out, "[%s] [mcsparse] %s\n", names[level < 0 ? 0 : (level > 4 ? 4 : level)], msg);
    std::fflush(out);
}
inline void log_error(const char* msg) { log_message(1, msg); }

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
