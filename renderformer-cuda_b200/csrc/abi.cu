// Library-level entry points of the C ABI: identification, status text, launch counter.
#include "common.cuh"

#include <cstdlib>

namespace rfk {
std::atomic<unsigned long long> g_launches{0};
bool g_pdl_enabled = [] { const char* e = getenv("RFK_PDL"); return !(e && e[0] == '0'); }();
}

extern "C" const char* rfk_version(void) { return "rfk 0.1 sm_100a"; }

extern "C" const char* rfk_status_string(int status) {
    switch (status) {
        case RFK_OK: return "ok";
        case RFK_EINVAL: return "invalid argument (null pointer, negative size or inconsistent shape)";
        case RFK_EUNSUPPORTED: return "shape or alignment not supported by this entry point";
        case RFK_ETOOBIG: return "size exceeds a fixed maximum of this entry point";
        case RFK_EKERNEL: return "a kernel gave up on a bounded device-side wait; its output is undefined";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown rfk status";
}

extern "C" unsigned long long rfk_launch_count(void) { return rfk::g_launches.load(std::memory_order_relaxed); }
