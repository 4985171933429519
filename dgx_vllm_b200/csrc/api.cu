// Utility entry points of the C ABI (status strings, version, capability probe, launch counter).
#include "common.cuh"

using namespace b200fp4;

extern "C" const char* b200fp4_get_error_string(int status) {
  switch (status) {
    case B200FP4_STATUS_SUCCESS: return "success";
    case B200FP4_STATUS_NOT_INITIALIZED: return "library not initialized";
    case B200FP4_STATUS_ALLOC_FAILED: return "workspace missing or too small";
    case B200FP4_STATUS_INVALID_VALUE: return "invalid argument (null pointer, bad size or misaligned pointer)";
    case B200FP4_STATUS_ARCH_MISMATCH: return "device is not compute capability 10.x (B200, sm_100a)";
    case B200FP4_STATUS_EXECUTION_FAILED: return "CUDA launch failed";
    case B200FP4_STATUS_INTERNAL_ERROR: return "internal error";
    case B200FP4_STATUS_NOT_SUPPORTED: return "shape or dtype not supported";
    default: return "unknown status";
  }
}

extern "C" int b200fp4_version(void) { return 100; }
extern "C" const char* b200fp4_version_string(void) { return "b200-nvfp4 0.1.0 (sm_100a)"; }

extern "C" int b200fp4_has_hardware_acceleration(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

extern "C" uint64_t b200fp4_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }
