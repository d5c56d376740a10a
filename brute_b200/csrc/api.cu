// Library-level entry points: error strings, capabilities, device status.
#include "common.cuh"

namespace bb { int tc5_status_bridge(); int at_status_bridge(); int sb_status_bridge(); int ly_status_bridge(); }

extern "C" const char* brute_b200_strerror(int code) {
    switch (code) {
        case BRUTE_OK:              return "ok";
        case BRUTE_ERR_INVALID_ARG: return "invalid argument";
        case BRUTE_ERR_MISALIGNED:  return "pointer or pitch is not aligned as required";
        case BRUTE_ERR_UNSUPPORTED: return "shape or dtype not supported by this path";
        case BRUTE_ERR_LAUNCH:      return "CUDA launch or runtime call failed";
        case BRUTE_ERR_WORKSPACE:   return "scratch buffer missing or too small";
        case BRUTE_ERR_DEVICE_WAIT: return "a bounded in-kernel wait gave up";
        case BRUTE_ERR_DRIVER:      return "a CUDA driver entry point is unavailable";
        default:                    return "unknown error";
    }
}

extern "C" uint32_t brute_b200_query_caps(void) {
    return BRUTE_CAP_SM100A | BRUTE_CAP_GEMM_POPC | BRUTE_CAP_GEMM_MMA_B1 | BRUTE_CAP_GEMM_TCGEN05 |
           BRUTE_CAP_ATTENTION;
}

extern "C" int brute_b200_device_status(void) {
    // every translation unit with bounded in-kernel waits keeps its own status word
    const int codes[4] = {bb::tc5_status_bridge(), bb::at_status_bridge(), bb::sb_status_bridge(), bb::ly_status_bridge()};
    for (int c : codes) if (c != BRUTE_OK) return c;
    return BRUTE_OK;
}
