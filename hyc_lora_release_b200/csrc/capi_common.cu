// Error strings and process-wide status of the C ABI.
#include "hyc_common.cuh"

static int g_last_cuda_error = 0;

extern "C" HYC_API void hyc_set_last_cuda_error(int e) { g_last_cuda_error = e; }
extern "C" HYC_API int hyc_last_cuda_error(void) { return g_last_cuda_error; }
extern "C" HYC_API int hyc_version(void) { return 100; }

extern "C" HYC_API const char* hyc_strerror(int code) {
  switch (code) {
    case HYC_OK: return "ok";
    case HYC_ERR_NULL: return "null pointer";
    case HYC_ERR_QBIT: return "q_bit must be 2, 4 or 8";
    case HYC_ERR_SHAPE: return "unsupported shape (see hyc.h for the divisibility and range rules)";
    case HYC_ERR_ALIGN: return "pointer or stride not aligned for vector access";
    case HYC_ERR_WORKSPACE: return "workspace missing or too small";
    case HYC_ERR_LAUNCH: return "CUDA launch failed (hyc_last_cuda_error() has the cudaError_t)";
    case HYC_ERR_CAPACITY: return "output capacity too small";
    case HYC_ERR_UNSUPPORTED: return "not supported by this build";
    default: return "unknown error";
  }
}
