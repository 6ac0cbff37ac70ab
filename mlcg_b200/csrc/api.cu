// Library-level entry points: error text, version, last CUDA error.
#include "common.cuh"

namespace mlcgb {
thread_local int g_last_cuda_error = 0;
}

extern "C" {

const char *mlcgb_strerror(int code) {
    switch (code) {
        case MLCGB_OK: return "ok";
        case MLCGB_E_ARG: return "invalid argument (null pointer, negative size or unsupported option)";
        case MLCGB_E_WORKSPACE: return "workspace too small";
        case MLCGB_E_LAUNCH: return "CUDA launch failed";
        case MLCGB_E_LIMIT: return "size beyond the supported limit";
        default: return "unknown error code";
    }
}

int mlcgb_last_cuda_error(void) { return mlcgb::g_last_cuda_error; }

int mlcgb_version(void) { return 100; }

}  // extern "C"
